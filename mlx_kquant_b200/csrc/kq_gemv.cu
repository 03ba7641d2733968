// Skinny-M quantized matmul (decode regime, at most 16 activation rows per
// weight matrix per task):
//   y[m, n] = sum_k x[m, k] * dequant(w)[n, k]
// replacing the reference's fused decode-then-dot CPU path
// (src/kquant_matmul.cpp:1104-1164 -> src/kquant_cpu_decode.cpp:1032-1065,
// 1254-1297) and, through GemvTask lists, its batched MoE decode
// (src/kquant_cpu_decode.cpp:1362-1527).
//
// The kernel is HBM-bound: every wire byte is read exactly once, with 16-byte
// loads issued one superblock ahead of their use.
//
// Work layout. A thread-block CLUSTER of S <= 8 CTAs owns 128 consecutive
// weight rows; CTA s of the cluster owns K-slice s, so even a 4096 x 4096
// matrix spreads over 256 CTAs while each CTA re-reads only its own 1/S of
// the activations. Inside a CTA the 8 warps own 16 rows each and walk the
// slice together; the slice's activations sit in shared memory (swizzled so
// the 16-byte fragment reads are conflict-free) and are shared by all warps.
// The S partial [128 x M] tiles meet through distributed shared memory:
// after a cluster barrier CTA s sums every S-th element over all peers and
// writes y. No scratch in global memory, no atomics, a fixed summation order.
//
// Inside a warp the 16 rows x 16 K products run on mma.sync m16n8k16 with the
// WEIGHTS as the A operand (lane (g, t) holds rows g and g+8) and 8 (or 16)
// activation rows as the B operand: the cost per weight does not grow with M up
// to 16, products are exact and accumulation is fp32.
//
//  * FAST (q4_k, fp16 activations): lane t of each quad owns sub-block pair
//    (2t, 2t+1) of the superblock: two 16-byte loads of quants per row, and only
//    its own two 6-bit scales to unpack. The A operand is the exact integer
//    sc*q (<= 63*15, exact in fp16), built by one HFMA2 from the 0x6400|q half
//    trick; a second MMA chain with A = mn gives sum(mn * x); the fp16 block
//    scales are applied in fp32 once per superblock:
//        y += d * sum(sc*q*x) - dmin * sum(mn*x).
//  * generic (every codec; f16 / bf16 / f32-as-bf16 activations): decode8<>
//    yields bit-exact fp32 weights, rounded to fp16 (fp16 activations) or split
//    into bf16 hi + lo (two MMAs), so the weight error stays below 2^-12.
#include <cooperative_groups.h>

#include <cstdlib>
#include <type_traits>

#include "kq_common.cuh"
#include "kq_launch.h"

namespace cg = cooperative_groups;

namespace kq {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kRowsPerCta = kGemvWarps * 16;
constexpr int kStageK = 1024;              // activations per row staged in shared memory at a time
constexpr int kStageChunks = kStageK / 8;  // 16-byte chunks per staged row
constexpr int kMaxSplit = 8;               // portable cluster size limit

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Programmatic dependent launch: a kernel launched with the programmatic-
// serialization attribute may start while its predecessor in the stream is
// still running; it must pass pdl_wait() before touching anything the
// predecessor writes (here: activations). Both are no-ops for plain launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Cluster-wide rendezvous without memory ordering: enough where a CTA only has to
// outlive its peers' reads of its shared memory (no data is handed over).
__device__ __forceinline__ void cluster_sync_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
}

// ---- activations in shared memory -------------------------------------------
// Row n of the stage holds kStageChunks 16-byte chunks (8 activations each).
// Chunk c of row n lives at slot c with its low three bits XOR-ed with bits 3-4
// of c and with the row parity, so the eight lanes that one LDS.128 phase
// serves (two rows x four quad lanes, whose chunks differ by 1 or by 8) always
// touch eight different 16-byte bank groups.
__device__ __forceinline__ int x_slot(int n, int c) {
  return n * kStageChunks + ((c & ~7) | ((c & 7) ^ ((c >> 3) & 3) ^ ((n & 1) << 2)));
}

// Stage activations [k0, k0 + kStageK) of the task's rows; rows >= m and
// columns >= k_end are zero. float input is rounded to bf16, as the reference's
// op does before its matmul (src/kquant_ops.cpp:159-168).
//
// PERM (the q4_k fast path, fp16 only) stores each chunk x0..x7 as
// x0 x2 x1 x3 x4 x6 x5 x7, the order in which the nibble unpacking yields
// weights, and also leaves, per row and 32-activation group, the group sum
// divided by 64 and split into an fp16 head and tail (sum / 64 = hi + lo to 2^-22) in `xsum`
// laid out [row][256-chunk][hi0..hi7 lo0..lo7].
template <typename XT, int NT, bool PERM>
__device__ __forceinline__ void stage_x(uint4* xs, __half* xsum, const GemvArgs& a, const int* s_xrow, int m, int k0,
                                        int k_end) {
  for (int idx = threadIdx.x; idx < NT * 8 * kStageChunks; idx += kGemvThreads) {
    const int n = idx / kStageChunks, c = idx % kStageChunks;
    const int k = k0 + 8 * c;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < m && k < k_end) {
      const XT* p = static_cast<const XT*>(a.x) + (long long)s_xrow[n] * a.x_row_stride + k;
      if constexpr (sizeof(XT) == 2) {
        v = __ldg(reinterpret_cast<const uint4*>(p));
      } else {
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p) + 1);
        v = make_uint4(pack_bf2(f0.x, f0.y), pack_bf2(f0.z, f0.w), pack_bf2(f1.x, f1.y), pack_bf2(f1.z, f1.w));
      }
    }
    if constexpr (PERM) {
      const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
      const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
      const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
      float sum = ((p0.x + p0.y) + (p1.x + p1.y)) + ((p2.x + p2.y) + (p3.x + p3.y));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // the four chunks of one 32-group sit in one aligned quad
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if ((c & 3) == 0) {
        // kept as sum / 64: thirty-two fp16 values can add up to 2^21, beyond fp16's range, and the
        // consumer multiplies the factor back in fp32
        sum *= 0.015625f;
        const __half hi = __float2half_rn(sum);
        const __half lo = __float2half_rn(sum - __half2float(hi));
        __half* dst = xsum + (n * (kStageK / 256) + (c >> 5)) * 16 + ((c >> 2) & 7);
        dst[0] = hi;
        dst[8] = lo;
      }
      v = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632), __byte_perm(v.z, v.w, 0x5410),
                     __byte_perm(v.z, v.w, 0x7632));
    }
    xs[x_slot(n, c)] = v;
  }
}

struct TaskView {
  const uint8_t* w;
  int m;
};

// Resolve this CTA's row group into shared memory. All CTAs of a cluster share
// blockIdx.x and blockIdx.z, so they take the same decision.
__device__ __forceinline__ bool resolve_task(const GemvArgs& a, int* s_xrow, int* s_yrow, TaskView& tv) {
  if (a.tasks != nullptr) {
    if (a.n_tasks_dev != nullptr && (int)blockIdx.z + a.task_offset >= *a.n_tasks_dev) return false;
    const GemvTask& t = a.tasks[blockIdx.z];
    tv.w = t.w;
    tv.m = t.m;
    if (threadIdx.x < 16) {
      s_xrow[threadIdx.x] = t.xrow[threadIdx.x];
      s_yrow[threadIdx.x] = t.yrow[threadIdx.x];
    }
  } else {
    const int r0 = blockIdx.z * 16;
    tv.w = a.w;
    tv.m = min(16, a.M - r0);
    if (threadIdx.x < 16) {
      s_xrow[threadIdx.x] = r0 + threadIdx.x;
      s_yrow[threadIdx.x] = r0 + threadIdx.x;
    }
  }
  __syncthreads();
  return tv.m > 0;
}

// ---- q4_k fast path pieces ---------------------------------------------------
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, __half2 b, __half2 c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), b, c);
  return *reinterpret_cast<uint32_t*>(&r);
}
// (a & mask) | magic as ONE three-input logic op. Written as C the two different
// constants become two instructions (a logic op carries a single immediate); with
// both constants in registers it is one.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t magic) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));
  return r;
}

struct Q4kLoad {  // what one lane consumes per superblock: header + its 32 quant bytes, for both of its rows
  uint4 hA, hB, qa0, qa1, qb0, qb1;
};

// Weight prefetch ring (fast path). Every warp owns kRing slots of one
// superblock x 16 rows (16 x 144 B) in dynamic shared memory and keeps up to
// kRing superblocks in flight with 16-byte cp.async copies - prefetch depth
// without register cost, and 16 fully used 144-byte segments per warp request.
constexpr int kRing = 2;
constexpr int kSlotBytes = 16 * 144;
constexpr int kRingBytesPerCta = kGemvWarps * kRing * kSlotBytes;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// wait until at most n (0..kRing-1) of this thread's copy groups are still pending
__device__ __forceinline__ void cp_async_wait(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
  }
}

// The 144 16-byte pieces of a slot are spread over the lanes: piece j = lane + 32 i
// is bytes [16 (j % 9), +16) of row j / 9. src_off / dst_off are fixed per lane.
struct Q4kRingLane {
  long long src_off[5];
  int dst_off[5];
};
__device__ __forceinline__ Q4kRingLane q4k_ring_lane(int lane, int row0, int n_rows, long long row_bytes) {
  Q4kRingLane r;
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const int j = lane + 32 * i;
    const int row = j / 9, piece = j % 9;
    r.src_off[i] = (long long)min(row0 + row, n_rows - 1) * row_bytes + piece * 16;
    r.dst_off[i] = row * 144 + piece * 16;
  }
  return r;
}
__device__ __forceinline__ void q4k_ring_issue(const Q4kRingLane& r, const uint8_t* w, uint8_t* slot, int sb,
                                               int lane) {
#pragma unroll
  for (int i = 0; i < 5; i++)
    if (i < 4 || lane < 16) cp_async16(slot + r.dst_off[i], w + r.src_off[i] + (long long)sb * 144);
  cp_async_commit();
}
__device__ __forceinline__ Q4kLoad q4k_ring_read(const uint8_t* slot, int g, int t) {
  const uint4* bA = reinterpret_cast<const uint4*>(slot + g * 144);
  const uint4* bB = reinterpret_cast<const uint4*>(slot + (g + 8) * 144);
  Q4kLoad l;
  l.hA = bA[0];
  l.hB = bB[0];
  l.qa0 = bA[1 + 2 * t];
  l.qa1 = bA[2 + 2 * t];
  l.qb0 = bB[1 + 2 * t];
  l.qb1 = bB[2 + 2 * t];
  return l;
}

// Scales of the lane's two sub-blocks (2t, 2t+1) of one row, ready for the
// unpacking below: lo nibbles become 1024+q and take (sc, -1024 sc); hi nibbles
// are left in place as 1024+16q and take (sc/16, -64 sc). All four constants and
// every product are exact in fp16 (sc <= 63, q <= 15).
struct Q4kRow {
  __half2 sc_lo, off_lo, sc_hi, off_hi;
  uint32_t mn;  // half2(mn[2t], mn[2t+1])
  float d, dmin;
};
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t two_bytes) {
  // (b0, b1) -> half2(b0, b1) exactly: 0x6400 | b is 1024 + b
  const uint32_t m = (two_bytes & 0xffu) | ((two_bytes & 0xff00u) << 8) | 0x64006400u;
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&m), __float2half2_rn(1024.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ Q4kRow q4k_row_prep(const uint4& hdr, int t) {
  Q4kRow r;
  r.d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
  r.dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
  // 6-bit pairs (src/kquant_cpu_decode.cpp:155-174), two sub-blocks at a time on 16-bit fields
  const int sh = 16 * (t & 1);
  const uint32_t u0 = (hdr.y >> sh) & 0xffffu, u1 = (hdr.z >> sh) & 0xffffu, u2 = (hdr.w >> sh) & 0xffffu;
  uint32_t sc2, mn2;
  if (t < 2) {
    sc2 = u0 & 0x3f3fu;
    mn2 = u1 & 0x3f3fu;
  } else {
    sc2 = (u2 & 0x0f0fu) | ((u0 >> 2) & 0x3030u);
    mn2 = ((u2 >> 4) & 0x0f0fu) | ((u1 >> 2) & 0x3030u);
  }
  const uint32_t sch = bytes_to_h2(sc2);
  const __half2 sc = *reinterpret_cast<const __half2*>(&sch);
  r.sc_lo = __low2half2(sc);
  r.off_lo = __hmul2(r.sc_lo, __float2half2_rn(-1024.f));
  r.sc_hi = __hmul2(__high2half2(sc), __float2half2_rn(0.0625f));
  r.off_hi = __hmul2(__high2half2(sc), __float2half2_rn(-64.f));
  r.mn = bytes_to_h2(mn2);
  return r;
}

// One superblock of the warp's 16 rows against the staged activations.
// sbl = index of the superblock inside the shared-memory stage; xoff[] are the
// lane's eight precomputed chunk slots of superblock 0 (see gemv_kernel).
template <int NT>
__device__ __forceinline__ void q4k_compute(const Q4kLoad& l, const uint4* xs, const __half* xsum, int sbl, int g,
                                            int t, const int (&xoff)[8], float (&fin)[NT][4]) {
  const Q4kRow ra = q4k_row_prep(l.hA, t), rb = q4k_row_prep(l.hB, t);
  const uint32_t wa[8] = {l.qa0.x, l.qa0.y, l.qa0.z, l.qa0.w, l.qa1.x, l.qa1.y, l.qa1.z, l.qa1.w};
  const uint32_t wb[8] = {l.qb0.x, l.qb0.y, l.qb0.z, l.qb0.w, l.qb1.x, l.qb1.y, l.qb1.z, l.qb1.w};
  float accq[NT][4], accm[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) accq[nt][i] = accm[nt][i] = 0.f;
  const uint4* xsb = xs + sbl * 32;
  const uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u, kMagic = 0x64006400u;
#pragma unroll
  for (int ip = 0; ip < 4; ip++) {
    uint4 x0[NT], x1[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      x0[nt] = xsb[xoff[ip] + nt * 8 * kStageChunks];      // sub-block 2t, activations 8ip..8ip+7
      x1[nt] = xsb[xoff[4 + ip] + nt * 8 * kStageChunks];  // sub-block 2t+1
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t Wa = wa[2 * ip + h], Wb = wb[2 * ip + h];
      const uint32_t Wa8 = Wa >> 8, Wb8 = Wb >> 8;
      // pairs (byte0, byte2) and (byte1, byte3): the staged activations are in the same order
      const uint32_t a0 = hfma2_u(and_or(Wa, kLo, kMagic), ra.sc_lo, ra.off_lo);
      const uint32_t a1 = hfma2_u(and_or(Wb, kLo, kMagic), rb.sc_lo, rb.off_lo);
      const uint32_t a2 = hfma2_u(and_or(Wa8, kLo, kMagic), ra.sc_lo, ra.off_lo);
      const uint32_t a3 = hfma2_u(and_or(Wb8, kLo, kMagic), rb.sc_lo, rb.off_lo);
      const uint32_t c0 = hfma2_u(and_or(Wa, kHi, kMagic), ra.sc_hi, ra.off_hi);
      const uint32_t c1 = hfma2_u(and_or(Wb, kHi, kMagic), rb.sc_hi, rb.off_hi);
      const uint32_t c2 = hfma2_u(and_or(Wa8, kHi, kMagic), ra.sc_hi, ra.off_hi);
      const uint32_t c3 = hfma2_u(and_or(Wb8, kHi, kMagic), rb.sc_hi, rb.off_hi);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        mma_f16(accq[nt], a0, a1, a2, a3, h ? x0[nt].z : x0[nt].x, h ? x0[nt].w : x0[nt].y);
        mma_f16(accq[nt], c0, c1, c2, c3, h ? x1[nt].z : x1[nt].x, h ? x1[nt].w : x1[nt].y);
      }
    }
  }
  // sum_s mn_s * xsum_s in one MMA: K slots 0-7 carry the fp16 heads of the eight
  // group sums, slots 8-15 their tails; the lane supplies mn of its sub-blocks 2t, 2t+1.
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const uint32_t* xq = reinterpret_cast<const uint32_t*>(xsum + ((nt * 8 + g) * (kStageK / 256) + sbl) * 16);
    mma_f16(accm[nt], ra.mn, rb.mn, ra.mn, rb.mn, xq[t], xq[4 + t]);
    // accm holds sum_s mn_s * xsum_s / 64 (the group sums are staged divided by 64)
    fin[nt][0] += ra.d * accq[nt][0] - ra.dmin * 64.f * accm[nt][0];
    fin[nt][1] += ra.d * accq[nt][1] - ra.dmin * 64.f * accm[nt][1];
    fin[nt][2] += rb.d * accq[nt][2] - rb.dmin * 64.f * accm[nt][2];
    fin[nt][3] += rb.d * accq[nt][3] - rb.dmin * 64.f * accm[nt][3];
  }
}

// ---- q4_k, one activation row (the decode case proper) --------------------------
// With a single token the eight columns of the B operand are free, and they are
// used to keep the eight sub-blocks of a superblock apart: column n of B holds
// x[k] for the K slots that belong to sub-block n and zero elsewhere. Lane (g, t)
// feeds slots of sub-block 2t (low nibbles) or 2t+1 (high nibbles), so it supplies
// real activations only when its column g is that sub-block and reads a block of
// zeros otherwise - a choice of base pointer made once per kernel. All sixteen
// MMAs of a superblock then accumulate into one fragment whose element
// (row, 2t + j) is sum_k (off_j + q_k) x_k over sub-block 2t + j: exactly the two
// sub-blocks whose 6-bit scales this lane unpacks. No per-weight arithmetic is
// left besides the three-input logic op that plants a nibble pair into fp16
// (0x6400 | q = 1024 + q for low nibbles, 0x5400 | q << 4 = 64 + q for high ones);
// the offsets leave with the fp32 group sums of x:
//   y += d * (sc0 (D0 - 1024 xs0) + sc1 (D1 - 64 xs1)) - dmin * (mn0 xs0 + mn1 xs1).
__device__ __forceinline__ float byte_to_float(uint32_t v, int byte) {
  // 0x4B0000bb is 2^23 + bb exactly
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 + byte)) - 8388608.f;
}

// qa0/qa1, qb0/qb1: the lane's 32 quant bytes of its two rows; hA/hB: the two block headers.
__device__ __forceinline__ void q4k_m1_compute(const uint4 hA, const uint4 hB, const uint4 qa0, const uint4 qa1,
                                               const uint4 qb0, const uint4 qb1, const uint4* plo, const uint4* phi,
                                               const float* xsum8, int t, const int (&xoff)[8], float& pA,
                                               float& pB) {
  const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
  const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
  const uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u, kM1024 = 0x64006400u, kM64 = 0x54005400u;
  // two independent accumulation chains: low-nibble MMAs only ever reach the even columns,
  // high-nibble MMAs the odd ones
  float accl[4] = {0.f, 0.f, 0.f, 0.f}, acch[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int ip = 0; ip < 4; ip++) {
    const uint4 x0 = plo[xoff[ip]];      // sub-block 2t, activations 8ip..8ip+7 (or zeros)
    const uint4 x1 = phi[xoff[4 + ip]];  // sub-block 2t+1
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t Wa = wa[2 * ip + h], Wb = wb[2 * ip + h];
      const uint32_t Wa8 = Wa >> 8, Wb8 = Wb >> 8;
      mma_f16(accl, and_or(Wa, kLo, kM1024), and_or(Wb, kLo, kM1024), and_or(Wa8, kLo, kM1024),
              and_or(Wb8, kLo, kM1024), h ? x0.z : x0.x, h ? x0.w : x0.y);
      mma_f16(acch, and_or(Wa, kHi, kM64), and_or(Wb, kHi, kM64), and_or(Wa8, kHi, kM64), and_or(Wb8, kHi, kM64),
              h ? x1.z : x1.x, h ? x1.w : x1.y);
    }
  }
  // the lane's two sub-blocks: 6-bit pairs (src/kquant_cpu_decode.cpp:155-174) on 16-bit fields
  const float2 xs = *reinterpret_cast<const float2*>(xsum8 + 2 * t);
  const int sh = 16 * (t & 1);
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const uint4 hdr = r ? hB : hA;
    const uint32_t u0 = (hdr.y >> sh) & 0xffffu, u1 = (hdr.z >> sh) & 0xffffu, u2 = (hdr.w >> sh) & 0xffffu;
    uint32_t sc2, mn2;
    if (t < 2) {
      sc2 = u0 & 0x3f3fu;
      mn2 = u1 & 0x3f3fu;
    } else {
      sc2 = (u2 & 0x0f0fu) | ((u0 >> 2) & 0x3030u);
      mn2 = ((u2 >> 4) & 0x0f0fu) | ((u1 >> 2) & 0x3030u);
    }
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // (d, dmin)
    const float t0 = fmaf(-1024.f, xs.x, accl[2 * r]), t1 = fmaf(-64.f, xs.y, acch[2 * r + 1]);
    const float u = fmaf(byte_to_float(sc2, 1), t1, byte_to_float(sc2, 0) * t0);
    const float v = fmaf(byte_to_float(mn2, 1), xs.y, byte_to_float(mn2, 0) * xs.x);
    float& p = r ? pB : pA;
    p = fmaf(dd.x, u, p);
    p = fmaf(-dd.y, v, p);
  }
}

// grid = (row groups of 128, S k-slices, 1); cluster = (1, S, 1). One activation row.
constexpr int kM1StageK = 2048;  // one token: 4 KB of activations cover eight superblocks per staging step
constexpr int kM1Chunks = kM1StageK / 8;
__global__ void __launch_bounds__(kGemvThreads, 3) gemv_q4k_m1_kernel(const GemvArgs a) {
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ __align__(16) uint4 xs1[kM1Chunks];  // the staged activations, pair-permuted and swizzled
  __shared__ __align__(16) uint4 xz[kM1Chunks];   // zeros: what a lane reads when its column is another sub-block
  __shared__ __align__(16) float xsumf[kM1StageK / 32];
  __shared__ float red[kRowsPerCta];
  extern __shared__ __align__(16) uint8_t dyn_smem[];

  cg::cluster_group cluster = cg::this_cluster();
  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;  // uniform over the cluster
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
  for (int i = threadIdx.x; i < kM1Chunks; i += kGemvThreads) xz[i] = make_uint4(0u, 0u, 0u, 0u);

  const int S = gridDim.y, slice = blockIdx.y;
  const int nchunks = a.K >> 8;
  const int per = (nchunks + S - 1) / S;
  const int ch0 = min(slice * per, nchunks), ch1 = min(ch0 + per, nchunks);

  // Weight ring: two slots per warp. Every loop step commits exactly one copy group (an empty one
  // once the slice is exhausted), so "all but the newest group" is always the superblock at hand.
  static_assert(kRing == 2, "the loop below toggles between two slots");
  uint8_t* ring = dyn_smem + warp * (kRing * kSlotBytes);
  const uint8_t* src[5];
  int dst[5];
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const int j = lane + 32 * i;
    const int row = j / 9, piece = j % 9;
    src[i] = tv.w + (long long)min(row0 + row, a.N - 1) * a.row_bytes + piece * 16 + (long long)ch0 * 144;
    dst[i] = row * 144 + piece * 16;
  }
  int issued = ch0;
  auto issue = [&](uint8_t* slot) {
    if (issued < ch1) {
#pragma unroll
      for (int i = 0; i < 5; i++) {
        if (i < 4 || lane < 16) cp_async16(slot + dst[i], src[i]);
        src[i] += 144;
      }
      issued++;
    }
    cp_async_commit();
  };
  issue(ring);
  issue(ring + kSlotBytes);
  pdl_launch_dependents();
  if (a.tasks == nullptr) pdl_wait();  // activations may come from the kernel before this one

  const uint4* xlo = (g == 2 * t) ? xs1 : xz;
  const uint4* xhi = (g == 2 * t + 1) ? xs1 : xz;
  int xoff[8];
#pragma unroll
  for (int i = 0; i < 8; i++) xoff[i] = x_slot(0, 8 * t + i);
  const __half* xrow = static_cast<const __half*>(a.x) + (long long)s_xrow[0] * a.x_row_stride;

  constexpr int kStageCh = kM1StageK / 256;
  float pA = 0.f, pB = 0.f;
  int soff = 0;  // byte offset of the current ring slot
  for (int sb = ch0; sb < ch1; sb++) {
    const int rel = sb - ch0;
    if (rel % kStageCh == 0) {
      if (rel != 0) __syncthreads();  // everyone is done with the previous stage
      {
        // one 16-byte chunk per thread: pair-permute it, and leave the fp32 sum of each 32-group
        static_assert(kM1Chunks == kGemvThreads, "one chunk per thread");
        const int c = threadIdx.x, k = sb * 256 + 8 * c;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (k < ch1 * 256) v = __ldg(reinterpret_cast<const uint4*>(xrow + k));  // nothing beyond this CTA's slice
        const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        float sum = ((p0.x + p0.y) + (p1.x + p1.y)) + ((p2.x + p2.y) + (p3.x + p3.y));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((c & 3) == 0) xsumf[c >> 2] = sum;
        xs1[x_slot(0, c)] = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632),
                                       __byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
      }
      __syncthreads();
    }
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncwarp();
    const uint4* bA = reinterpret_cast<const uint4*>(ring + soff + g * 144);
    const uint4* bB = reinterpret_cast<const uint4*>(ring + soff + (g + 8) * 144);
    const uint4 hA = bA[0], hB = bB[0];
    const uint4 qa0 = bA[1 + 2 * t], qa1 = bA[2 + 2 * t], qb0 = bB[1 + 2 * t], qb1 = bB[2 + 2 * t];
    __syncwarp();  // the slot is free again
    issue(ring + soff);
    soff ^= kSlotBytes;
    const int sbl = rel % kStageCh;
    q4k_m1_compute(hA, hB, qa0, qa1, qb0, qb1, xlo + sbl * 32, xhi + sbl * 32, xsumf + sbl * 8, t, xoff, pA, pB);
  }
  // the four lanes of a quad hold the four sub-block pairs of the same two rows
  pA += __shfl_xor_sync(0xffffffffu, pA, 1);
  pB += __shfl_xor_sync(0xffffffffu, pB, 1);
  pA += __shfl_xor_sync(0xffffffffu, pA, 2);
  pB += __shfl_xor_sync(0xffffffffu, pB, 2);
  if (t == 0) {
    red[warp * 16 + g] = pA;
    red[warp * 16 + g + 8] = pB;
  }
  cluster.sync();
  const float* peer[kMaxSplit];
#pragma unroll
  for (int s = 0; s < kMaxSplit; s++) peer[s] = s < S ? cluster.map_shared_rank(red, s) : red;
  const int cta_row0 = blockIdx.x * kRowsPerCta;
  for (int idx = slice + S * threadIdx.x; idx < kRowsPerCta; idx += S * kGemvThreads) {
    if (cta_row0 + idx < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxSplit; s++)
        if (s < S) sum += peer[s][idx];
      static_cast<__half*>(a.y)[(long long)s_yrow[0] * a.y_row_stride + cta_row0 + idx] = __float2half_rn(sum);
    }
  }
  cluster_sync_relaxed();  // peers may still be reading this CTA's partial sums
}

// ---- one activation row, small matrices ------------------------------------------
// For a matrix of a few MB the launch is a latency chain, not a stream: what counts is how
// little is left to do once the activations exist. Here a CTA of four warps owns 16 rows and
// the warps split K between them, so partial sums meet in the CTA's own shared memory (no
// cluster, no second barrier), ALL of a CTA's weights are in flight before it waits for the
// preceding kernel, and a CTA is small enough (128 threads, ~46 KB) that the whole grid of the
// next launch fits beside the running one and has its weights on chip when its turn comes.
// grid = (ceil(N / 16), 1, 1). K <= kRowsMaxK: the activations are staged whole.
constexpr int kRowsWarps = 4, kRowsThreads = 32 * kRowsWarps, kRowsDepth = 4, kRowsMaxK = 8192;
constexpr int kRowsRingBytes = kRowsWarps * kRowsDepth * kSlotBytes;
static inline int rows_dyn_smem(int K) { return kRowsRingBytes + K * 2 + (K / 32) * 4; }

__global__ void __launch_bounds__(kRowsThreads, 4) gemv_q4k_m1_rows_kernel(const GemvArgs a) {
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ __align__(16) uint4 xz[32];  // zeros: what a lane reads when its column is another sub-block
  __shared__ float red[kRowsWarps * 16];
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  const int nchunks = a.K >> 8;
  uint4* xs1 = reinterpret_cast<uint4*>(dyn_smem + kRowsRingBytes);  // pair-permuted, swizzled activations
  float* xsumf = reinterpret_cast<float*>(dyn_smem + kRowsRingBytes + nchunks * 512);

  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  if (threadIdx.x < 32) xz[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);

  const int per = (nchunks + kRowsWarps - 1) / kRowsWarps;
  const int ch0 = min(warp * per, nchunks), ch1 = min(ch0 + per, nchunks);

  // Per-warp ring of kRowsDepth superblocks x 16 rows. Every issue() commits exactly one copy
  // group (an empty one past the slice), so "all but the newest kRowsDepth - 1" is always the
  // superblock at hand.
  uint8_t* ring = dyn_smem + warp * (kRowsDepth * kSlotBytes);
  const uint8_t* src[5];
  int dst[5];
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const int j = lane + 32 * i;
    const int row = j / 9, piece = j % 9;
    src[i] = tv.w + (long long)min(row0 + row, a.N - 1) * a.row_bytes + piece * 16 + (long long)ch0 * 144;
    dst[i] = row * 144 + piece * 16;
  }
  int issued = ch0;
  auto issue = [&](uint8_t* slot) {
    if (issued < ch1) {
#pragma unroll
      for (int i = 0; i < 5; i++) {
        if (i < 4 || lane < 16) cp_async16(slot + dst[i], src[i]);
        src[i] += 144;
      }
      issued++;
    }
    cp_async_commit();
  };
#pragma unroll
  for (int d = 0; d < kRowsDepth; d++) issue(ring + d * kSlotBytes);
  pdl_launch_dependents();
  if (a.tasks == nullptr) pdl_wait();  // activations may come from the kernel before this one

  {
    // all of K: pair-permute each 16-byte chunk and leave the fp32 sum of each 32-group.
    // All loads are issued before the first use: one L2 round trip, not one per iteration.
    const __half* xrow = static_cast<const __half*>(a.x) + (long long)s_xrow[0] * a.x_row_stride;
    constexpr int kIt = kRowsMaxK / 8 / kRowsThreads;
    uint4 xv[kIt];
#pragma unroll
    for (int it = 0; it < kIt; it++) {
      const int c = threadIdx.x + kRowsThreads * it;
      xv[it] = make_uint4(0u, 0u, 0u, 0u);
      if (c < nchunks * 32) xv[it] = __ldg(reinterpret_cast<const uint4*>(xrow + 8 * c));
    }
#pragma unroll
    for (int it = 0; it < kIt; it++) {
      const int c = threadIdx.x + kRowsThreads * it;
      if (c < nchunks * 32) {  // uniform over a warp: 32 chunks per superblock
        const uint4 v = xv[it];
        const float2 p0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 p1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 p3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        float sum = ((p0.x + p0.y) + (p1.x + p1.y)) + ((p2.x + p2.y) + (p3.x + p3.y));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((c & 3) == 0) xsumf[c >> 2] = sum;
        xs1[x_slot(0, c)] = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632),
                                       __byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
      }
    }
  }
  __syncthreads();

  const uint4* xlo = (g == 2 * t) ? xs1 : xz;
  const uint4* xhi = (g == 2 * t + 1) ? xs1 : xz;
  const int lo_step = (g == 2 * t) ? 32 : 0, hi_step = (g == 2 * t + 1) ? 32 : 0;
  int xoff[8];
#pragma unroll
  for (int i = 0; i < 8; i++) xoff[i] = x_slot(0, 8 * t + i);

  float pA = 0.f, pB = 0.f;
  for (int sb = ch0; sb < ch1; sb++) {
    const int rel = sb - ch0;
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kRowsDepth - 1) : "memory");
    __syncwarp();
    uint8_t* slot = ring + (rel % kRowsDepth) * kSlotBytes;
    const uint4* bA = reinterpret_cast<const uint4*>(slot + g * 144);
    const uint4* bB = reinterpret_cast<const uint4*>(slot + (g + 8) * 144);
    const uint4 hA = bA[0], hB = bB[0];
    const uint4 qa0 = bA[1 + 2 * t], qa1 = bA[2 + 2 * t], qb0 = bB[1 + 2 * t], qb1 = bB[2 + 2 * t];
    __syncwarp();  // the slot is free again
    issue(slot);
    q4k_m1_compute(hA, hB, qa0, qa1, qb0, qb1, xlo + sb * lo_step, xhi + sb * hi_step, xsumf + sb * 8, t, xoff, pA,
                   pB);
  }
  // the four lanes of a quad hold the four sub-block pairs of the same two rows
  pA += __shfl_xor_sync(0xffffffffu, pA, 1);
  pB += __shfl_xor_sync(0xffffffffu, pB, 1);
  pA += __shfl_xor_sync(0xffffffffu, pA, 2);
  pB += __shfl_xor_sync(0xffffffffu, pB, 2);
  if (t == 0) {
    red[warp * 16 + g] = pA;
    red[warp * 16 + g + 8] = pB;
  }
  __syncthreads();
  if (threadIdx.x < 16 && row0 + threadIdx.x < a.N) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kRowsWarps; w++) sum += red[w * 16 + threadIdx.x];
    static_cast<__half*>(a.y)[(long long)s_yrow[0] * a.y_row_stride + row0 + threadIdx.x] = __float2half_rn(sum);
  }
}

// ---- one activation row on the integer dot-product pipe ------------------------------
// With a single activation row the tensor-core formulations above waste seven of eight MMA
// columns, and the legacy tensor pipe, not HBM, bounds them. Here the products run on dp4a
// instead: the activations of each 32-group are quantized once per CTA to 16-bit integers with
// the group's own scale (xi = rint(x * 32767 / max|x|), |error| <= 2^-16 of the group maximum -
// far below the fp16 / bf16 rounding the activations already carry) and stored as two int8 planes
// (xi = 256 xh + xl). One three-input logic op then yields FOUR weights (W & 0x0f0f0f0f), one
// dp4a per plane multiplies them; the integer sums are exact, and scale, 6-bit sub-block scales,
// d and dmin are applied in fp32 per sub-block (src/kquant_cpu_decode.cpp:155-174, 177-202).
// Thread = weight row (a warp owns 32 rows), the eight warps of a CTA split K and meet in shared
// memory. Works for fp16, bf16 and float activations alike (float is rounded to bf16 first, as
// the op does, src/kquant_ops.cpp:159-168).
constexpr int kDpWarps = 8, kDpThreads = 32 * kDpWarps, kDpRows = 32, kDpSlot = kDpRows * 144;
constexpr int kDpMaxK = 16384;
static inline int dp_dyn_smem(int K, int D) { return kDpWarps * D * kDpSlot + 2 * K + 2 * (K / 32) * 4; }

template <typename XT>
__global__ void __launch_bounds__(kDpThreads, 2) gemv_q4k_m1_dp4a_kernel(const GemvArgs a, const int D, const int rpc) {
  using OT = typename std::conditional<std::is_same<XT, __half>::value, __half, __nv_bfloat16>::type;
  __shared__ float red[kDpWarps][kDpRows];
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nchunks = a.K >> 8;
  uint32_t* XH = reinterpret_cast<uint32_t*>(dyn_smem + kDpWarps * D * kDpSlot);  // high bytes, four per word
  uint32_t* XL = XH + a.K / 4;                                                    // low bytes
  float* SG = reinterpret_cast<float*>(XL + a.K / 4);                             // scale of each 32-group
  float* XS = SG + a.K / 32;                                                      // sum of each 32-group
  // rpc <= 32 rows per CTA: a grid that covers all SMs when N / 32 would leave some idle
  const int row0 = blockIdx.x * rpc;
  const int row_end = min(row0 + rpc, a.N);
  const int per = (nchunks + kDpWarps - 1) / kDpWarps;
  const int ch0 = min(warp * per, nchunks), ch1 = min(ch0 + per, nchunks);

  // Per-warp ring of D superblocks x 32 rows; every issue() commits exactly one copy group.
  uint8_t* ring = dyn_smem + warp * D * kDpSlot;
  const uint8_t* src[9];
#pragma unroll
  for (int i = 0; i < 9; i++) {
    const int j = lane + 32 * i;  // 288 16-byte pieces per superblock, contiguous in the slot
    src[i] = a.w + (long long)min(row0 + j / 9, row_end - 1) * a.row_bytes + (long long)ch0 * 144 + (j % 9) * 16;
  }
  int issued = ch0;
  auto issue = [&](uint8_t* slot) {
    if (issued < ch1) {
#pragma unroll
      for (int i = 0; i < 9; i++) {
        cp_async16(slot + 16 * (lane + 32 * i), src[i]);
        src[i] += 144;
      }
      issued++;
    }
    cp_async_commit();
  };
  for (int d = 0; d < D; d++) issue(ring + d * kDpSlot);
  pdl_launch_dependents();
  pdl_wait();  // activations may come from the kernel before this one

  {
    // quantize all of K: eight activations per thread and step, four threads per 32-group
    const XT* xrow = static_cast<const XT*>(a.x);
    for (int c = threadIdx.x; c < a.K / 8; c += kDpThreads) {
      float v[8];
      if constexpr (std::is_same<XT, float>::value) {
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(xrow + 8 * c));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(xrow + 8 * c) + 1);
        const float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __bfloat162float(__float2bfloat16_rn(f[i]));
      } else {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(xrow + 8 * c));
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float2 f;
          if constexpr (std::is_same<XT, __half>::value) f = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
          else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[i]));
          v[2 * i] = f.x;
          v[2 * i + 1] = f.y;
        }
      }
      float amax = 0.f, sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        amax = fmaxf(amax, fabsf(v[i]));
        sum += v[i];
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      const bool finite = amax > 0.f && amax < INFINITY;
      // the reciprocal need not be exact: xi * scale reproduces v to ~1e-7 either way
      const float inv = finite ? 32767.f * __frcp_rn(amax) : 0.f;
      uint32_t h[2] = {0u, 0u}, l[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int xi = __float2int_rn(v[i] * inv);
        h[i >> 2] |= ((uint32_t)(xi >> 8) & 0xffu) << (8 * (i & 3));
        l[i >> 2] |= ((uint32_t)xi & 0xffu) << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(XH + 2 * c) = make_uint2(h[0], h[1]);
      *reinterpret_cast<uint2*>(XL + 2 * c) = make_uint2(l[0], l[1]);
      if ((c & 3) == 0) {
        // a group holding inf / nan keeps them: the scale carries the non-finite value into the sum
        SG[c >> 2] = finite ? amax * (1.f / 32767.f) : (amax > 0.f ? amax : 0.f);
        XS[c >> 2] = sum;
      }
    }
  }
  __syncthreads();

  float y = 0.f;
  for (int sb = ch0; sb < ch1; sb++) {
    const int rel = sb - ch0;
    cp_async_wait(D - 1);
    __syncwarp();
    uint8_t* slot = ring + (rel % D) * kDpSlot;
    const uint4* blk = reinterpret_cast<const uint4*>(slot + lane * 144);
    const uint4 hdr = blk[0];
    uint4 q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = blk[1 + i];
    __syncwarp();  // the slot is free again
    issue(slot);
    // eight 6-bit (scale, min) pairs from twelve bytes, four at a time
    const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
    const uint32_t scl = u0 & 0x3f3f3f3fu, mnl = u1 & 0x3f3f3f3fu;
    const uint32_t sch = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
    const uint32_t mnh = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
    const uint4* xh4 = reinterpret_cast<const uint4*>(XH + sb * 64);
    const uint4* xl4 = reinterpret_cast<const uint4*>(XL + sb * 64);
    const float4* sg4 = reinterpret_cast<const float4*>(SG + sb * 8);
    const float4* xs4 = reinterpret_cast<const float4*>(XS + sb * 8);
    const float4 sga = sg4[0], sgb = sg4[1], xsa = xs4[0], xsb = xs4[1];
    const float sg[8] = {sga.x, sga.y, sga.z, sga.w, sgb.x, sgb.y, sgb.z, sgb.w};
    const float xs[8] = {xsa.x, xsa.y, xsa.z, xsa.w, xsb.x, xsb.y, xsb.z, xsb.w};
    float t1 = 0.f, t2 = 0.f;
#pragma unroll
    for (int p = 0; p < 4; p++) {
      // 32 bytes: low nibbles are sub-block 2p, high nibbles sub-block 2p + 1, weights in natural order
      const uint32_t w[8] = {q[2 * p].x, q[2 * p].y, q[2 * p].z, q[2 * p].w,
                             q[2 * p + 1].x, q[2 * p + 1].y, q[2 * p + 1].z, q[2 * p + 1].w};
      const uint4 ha0 = xh4[4 * p], ha1 = xh4[4 * p + 1], hb0 = xh4[4 * p + 2], hb1 = xh4[4 * p + 3];
      const uint4 la0 = xl4[4 * p], la1 = xl4[4 * p + 1], lb0 = xl4[4 * p + 2], lb1 = xl4[4 * p + 3];
      const uint32_t xha[8] = {ha0.x, ha0.y, ha0.z, ha0.w, ha1.x, ha1.y, ha1.z, ha1.w};
      const uint32_t xhb[8] = {hb0.x, hb0.y, hb0.z, hb0.w, hb1.x, hb1.y, hb1.z, hb1.w};
      const uint32_t xla[8] = {la0.x, la0.y, la0.z, la0.w, la1.x, la1.y, la1.z, la1.w};
      const uint32_t xlb[8] = {lb0.x, lb0.y, lb0.z, lb0.w, lb1.x, lb1.y, lb1.z, lb1.w};
      int ah_lo = 0, ah_hi = 0;
      unsigned al_lo = 0u, al_hi = 0u;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        // high nibbles stay where they are: 16 q as an unsigned byte, the 1/16 goes into the scale
        const uint32_t lo = w[j] & 0x0f0f0f0fu, hi = w[j] & 0xf0f0f0f0u;
        ah_lo = __dp4a((int)lo, (int)xha[j], ah_lo);
        al_lo = __dp4a(lo, xla[j], al_lo);
        asm("dp4a.u32.s32 %0, %1, %2, %3;\n" : "=r"(ah_hi) : "r"(hi), "r"(xhb[j]), "r"(ah_hi));
        al_hi = __dp4a(hi, xlb[j], al_hi);
      }
      const float f_lo = (float)(ah_lo * 256 + (int)al_lo), f_hi = (float)(ah_hi * 256 + (int)al_hi) * 0.0625f;
      const float sc_lo = byte_to_float(p < 2 ? scl : sch, 2 * (p & 1)), sc_hi = byte_to_float(p < 2 ? scl : sch, 2 * (p & 1) + 1);
      const float mn_lo = byte_to_float(p < 2 ? mnl : mnh, 2 * (p & 1)), mn_hi = byte_to_float(p < 2 ? mnl : mnh, 2 * (p & 1) + 1);
      t1 = fmaf(sc_lo * sg[2 * p], f_lo, t1);
      t1 = fmaf(sc_hi * sg[2 * p + 1], f_hi, t1);
      t2 = fmaf(mn_lo, xs[2 * p], t2);
      t2 = fmaf(mn_hi, xs[2 * p + 1], t2);
    }
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // (d, dmin)
    y = fmaf(dd.x, t1, y);
    y = fmaf(-dd.y, t2, y);
  }
  red[warp][lane] = y;
  __syncthreads();
  if (warp == 0 && row0 + lane < row_end) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kDpWarps; w++) sum += red[w][lane];
    OT* out = static_cast<OT*>(a.y) + row0 + lane;
    if constexpr (std::is_same<OT, __half>::value) *out = __float2half_rn(sum);
    else *out = __float2bfloat16_rn(sum);
  }
}

// ---- the kernel ---------------------------------------------------------------
// grid = (row groups of 128, S k-slices, tasks); cluster = (1, S, 1).
template <int C, int A, typename XT, int NT, bool FAST>
__global__ void __launch_bounds__(kGemvThreads) gemv_kernel(const GemvArgs a) {
  constexpr bool kHalf = std::is_same<XT, __half>::value;
  using OT = typename std::conditional<kHalf, __half, __nv_bfloat16>::type;
  constexpr int WPB = wpb_of(C), BPB = bpb_of(C);
  constexpr int kTile = NT * 8 * kRowsPerCta;  // floats in one CTA's partial tile
  constexpr bool kIq = (C == IQ4_NL || C == IQ4_XS || C == IQ2_XXS);
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ __align__(16) uint4 xs[NT * 8 * kStageChunks];
  __shared__ float red[kTile];
  __shared__ __align__(16) uint8_t s_tabs[kIq ? kIqSmemBytes : 16];
  __shared__ __align__(16) __half xsum[FAST ? NT * 8 * (kStageK / 256) * 16 : 8];

  cg::cluster_group cluster = cg::this_cluster();
  IqTables tabs = global_iq_tables();
  if constexpr (kIq) {
    tabs = stage_iq_tables(s_tabs, threadIdx.x, kGemvThreads);
  }
  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;  // uniform over the cluster

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
  const uint8_t* pA = tv.w + (long long)min(row0 + g, a.N - 1) * a.row_bytes;
  const uint8_t* pB = tv.w + (long long)min(row0 + g + 8, a.N - 1) * a.row_bytes;

  // this CTA's K-slice, in 256-weight chunks
  const int S = gridDim.y, slice = blockIdx.y;
  const int nchunks = (a.K + 255) >> 8;
  const int per = (nchunks + S - 1) / S;
  const int ch0 = min(slice * per, nchunks), ch1 = min(ch0 + per, nchunks);

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[nt][i] = 0.f;

  // fast path: the lane's chunk slots inside superblock 0 of the stage, row g
  // (sub-block 2t: chunks 8t+ip, sub-block 2t+1: chunks 8t+4+ip)
  int xoff[8];
#pragma unroll
  for (int i = 0; i < 8; i++) xoff[i] = x_slot(g, 8 * t + i);

  constexpr int kStageCh = kStageK / 256;  // 256-weight chunks per stage
  if constexpr (FAST) {
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    uint8_t* ring = dyn_smem + warp * (kRing * kSlotBytes);
    const Q4kRingLane rl = q4k_ring_lane(lane, row0, a.N, a.row_bytes);
    // Weights never depend on the preceding kernel: start streaming them before
    // anything else, up to kRing superblocks deep.
    int issued = ch0;
    for (int d = 0; d < kRing && issued < ch1; d++, issued++)
      q4k_ring_issue(rl, tv.w, ring + d * kSlotBytes, issued, lane);
    // Every CTA of this grid is resident by the time all of them have said so;
    // the next kernel in the stream may then start streaming ITS weights.
    pdl_launch_dependents();
    if (a.tasks == nullptr) pdl_wait();  // activations may come from the kernel before this one
    for (int sb = ch0; sb < ch1; sb++) {
      const int rel = sb - ch0;
      if (rel % kStageCh == 0) {
        if (rel != 0) __syncthreads();  // everyone is done with the previous stage
        stage_x<XT, NT, true>(xs, xsum, a, s_xrow, tv.m, sb * 256, a.K);
        __syncthreads();
      }
      cp_async_wait(issued - sb - 1);
      __syncwarp();
      const Q4kLoad cur = q4k_ring_read(ring + (rel % kRing) * kSlotBytes, g, t);
      __syncwarp();  // the slot is free again
      if (issued < ch1) {
        q4k_ring_issue(rl, tv.w, ring + (rel % kRing) * kSlotBytes, issued, lane);
        issued++;
      }
      q4k_compute<NT>(cur, xs, xsum, rel % kStageCh, g, t, xoff, acc);
    }
  } else {
    pdl_launch_dependents();
    if (a.tasks == nullptr) pdl_wait();
    for (int cs = ch0; cs < ch1; cs += kStageCh) {
      const int ce = min(cs + kStageCh, ch1);
      if (cs != ch0) __syncthreads();  // everyone is done with the previous stage
      stage_x<XT, NT, false>(xs, xsum, a, s_xrow, tv.m, cs * 256, a.K);
      __syncthreads();
      const int ngroups = a.K / 32;
      const int g_end = min(ce * 8, ngroups);
#pragma unroll 2
      for (int gi = cs * 8; gi < g_end; gi++) {
        long long boff;
        int oct;
        boff = block_of<C>(32ll * gi) * BPB;   // group gi = weights 32 gi .. 32 gi + 31 of the row
        oct = octet_of<C>(32ll * gi) + t;
        float va[8], vb[8];
        decode8<C, A>(pA + boff, oct, va, tabs);
        decode8<C, A>(pB + boff, oct, vb, tabs);
        const int c = (gi - cs * 8) * 4 + t;
        uint4 xb[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) xb[nt] = xs[x_slot(nt * 8 + g, c)];
        uint32_t ha[4], hb[4];
        if constexpr (kHalf) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            ha[i] = pack_h2(va[2 * i], va[2 * i + 1]);
            hb[i] = pack_h2(vb[2 * i], vb[2 * i + 1]);
          }
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            mma_f16(acc[nt], ha[0], hb[0], ha[1], hb[1], xb[nt].x, xb[nt].y);
            mma_f16(acc[nt], ha[2], hb[2], ha[3], hb[3], xb[nt].z, xb[nt].w);
          }
        } else {
          uint32_t la[4], lb[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h1 = __floats2bfloat162_rn(va[2 * i], va[2 * i + 1]);
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(vb[2 * i], vb[2 * i + 1]);
            ha[i] = *reinterpret_cast<const uint32_t*>(&h1);
            hb[i] = *reinterpret_cast<const uint32_t*>(&h2);
            la[i] = pack_bf2(va[2 * i] - __low2float(h1), va[2 * i + 1] - __high2float(h1));
            lb[i] = pack_bf2(vb[2 * i] - __low2float(h2), vb[2 * i + 1] - __high2float(h2));
          }
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            mma_bf16(acc[nt], ha[0], hb[0], ha[1], hb[1], xb[nt].x, xb[nt].y);
            mma_bf16(acc[nt], la[0], lb[0], la[1], lb[1], xb[nt].x, xb[nt].y);
            mma_bf16(acc[nt], ha[2], hb[2], ha[3], hb[3], xb[nt].z, xb[nt].w);
            mma_bf16(acc[nt], la[2], lb[2], la[3], lb[3], xb[nt].z, xb[nt].w);
          }
        }
      }
    }
  }
  // ---- partial tile -> shared memory, [token][row] so that y stores are contiguous
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int tok = nt * 8 + 2 * t + (i & 1);
      const int row = warp * 16 + g + 8 * (i >> 1);
      red[tok * kRowsPerCta + row] = acc[nt][i];
    }
  cluster.sync();
  // CTA `slice` finishes elements slice, slice + S, ... of the tile: fixed order over the S peers
  const float* peer[kMaxSplit];
#pragma unroll
  for (int s = 0; s < kMaxSplit; s++) peer[s] = s < S ? cluster.map_shared_rank(red, s) : red;
  const int cta_row0 = blockIdx.x * kRowsPerCta;
  for (int idx = slice + S * threadIdx.x; idx < kTile; idx += S * kGemvThreads) {
    const int tok = idx / kRowsPerCta, row = idx % kRowsPerCta;
    if (tok < tv.m && cta_row0 + row < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxSplit; s++)
        if (s < S) sum += peer[s][idx];
      OT* y = static_cast<OT*>(a.y) + (long long)s_yrow[tok] * a.y_row_stride + cta_row0 + row;
      if (a.bias != nullptr) sum += (float)static_cast<const OT*>(a.bias)[cta_row0 + row];
      if constexpr (kHalf) {
        if (a.out_bf16) {  // rows that were bf16 / f32 before their exact conversion to fp16
          const float rs = a.row_scale ? a.row_scale[s_xrow[tok]] : 1.f;
          *reinterpret_cast<__nv_bfloat16*>(y) = __float2bfloat16_rn(sum * rs);
        } else {
          *y = __float2half_rn(sum);
        }
      } else {
        *y = __float2bfloat16_rn(sum);
      }
    }
  }
  cluster_sync_relaxed();  // peers may still be reading this CTA's tile
}

// ---- table-driven kernel for the IQ codecs (iq4_xs, iq2_xxs) ------------------------
// Same work layout as gemv_kernel (cluster split-K, 8 warps x 16 rows, weights through
// a per-warp cp.async ring, activations staged in swizzled shared memory), but the A
// fragments come from lookup tables in shared memory that already hold the values in
// the multiplicand type:
//   iq4_xs   256 entries: byte -> pair (LUT[low nibble], LUT[high nibble])
//            (src/kquant_cpu_decode.cpp:441-465, kvalues_iq4nl)
//   iq2_xxs  256 entries: grid index -> its eight lattice values; 128 entries: 7-bit sign
//            index -> four words of sign-bit masks to XOR in
//            (src/kquant_cpu_decode.cpp:557-584, iq2xxs_grid / ksigns_iq2xs)
// The four lanes of a quad work on the same 32-weight group, so two MMAs give the
// exact integer dot products of that group for the warp's 16 rows, and the group's
// fp32 scale (d * (ls - 32), resp. d * (0.5 + s) / 4) is applied once per group.
// Block sizes (136 and 66 bytes) are not multiples of 16: the ring copies the
// 16-byte-aligned window around each block and readers add the block's phase.
template <int C>
struct IqGeom;
template <>
struct IqGeom<IQ4_XS> {
  static constexpr int kBpb = 136, kPieces = 9, kStride = 160;
};
template <>
struct IqGeom<IQ2_XXS> {
  static constexpr int kBpb = 66, kPieces = 5, kStride = 96;
};

template <typename MT>
__device__ __forceinline__ uint32_t pack_mt(float a, float b) {
  if constexpr (std::is_same<MT, __half>::value) return pack_h2(a, b);
  else return pack_bf2(a, b);
}

template <int C, typename XT, int NT>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_iq_kernel(const GemvArgs a) {
  constexpr bool kHalf = std::is_same<XT, __half>::value;
  using MT = typename std::conditional<kHalf, __half, __nv_bfloat16>::type;
  using G = IqGeom<C>;
  constexpr int kSlot = 16 * G::kStride;
  constexpr int kTile = NT * 8 * kRowsPerCta;
  __shared__ int s_xrow[16], s_yrow[16];
  __shared__ __align__(16) uint4 xs[NT * 8 * kStageChunks];
  __shared__ float red[kTile];
  __shared__ __align__(16) uint32_t tab[C == IQ4_XS ? 256 : 256 * 2];
  extern __shared__ __align__(16) uint8_t dyn_smem[];

  cg::cluster_group cluster = cg::this_cluster();
  // tables, in the multiplicand type
  if constexpr (C == IQ4_XS) {
    for (int b = threadIdx.x; b < 256; b += kGemvThreads)
      tab[b] = pack_mt<MT>((float)kq_tab_iq4nl[b & 15], (float)kq_tab_iq4nl[b >> 4]);
  } else {
    // the lattice as it is: 256 x 8 bytes; bytes become multiplicands with the magic-number trick
    for (int i = threadIdx.x; i < 256; i += kGemvThreads)
      reinterpret_cast<unsigned long long*>(tab)[i] = kq_tab_iq2xxs_grid[i];
  }
  // iq4_xs, fp16: the 16-entry level table in four registers, looked up with byte permutes
  uint32_t T[4] = {0u, 0u, 0u, 0u};
  if constexpr (C == IQ4_XS && kHalf) {
#pragma unroll
    for (int i = 0; i < 16; i++) T[i >> 2] |= ((uint32_t)(uint8_t)kq_tab_iq4nl[i]) << (8 * (i & 3));
  }
  TaskView tv;
  if (!resolve_task(a, s_xrow, s_yrow, tv)) return;  // uniform over the cluster; also publishes the tables

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
  const int S = gridDim.y, slice = blockIdx.y;
  const int nchunks = a.K >> 8;
  const int per = (nchunks + S - 1) / S;
  const int ch0 = min(slice * per, nchunks), ch1 = min(ch0 + per, nchunks);

  // ring: the lane's pieces of a slot (piece j = lane + 32 i is bytes [16 (j % P), +16) of row j / P)
  constexpr int kPerLane = (16 * G::kPieces + 31) / 32;
  uint8_t* ring = dyn_smem + warp * (kRing * kSlot);
  const uint8_t* src[kPerLane];
  int dst[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; i++) {
    const int j = min(lane + 32 * i, 16 * G::kPieces - 1);
    const int row = j / G::kPieces, piece = j % G::kPieces;
    src[i] = tv.w + (long long)min(row0 + row, a.N - 1) * a.row_bytes + piece * 16;
    dst[i] = row * G::kStride + piece * 16;
  }
  int issued = ch0;
  auto issue = [&](uint8_t* slot) {
    if (issued < ch1) {
      const long long base = ((long long)issued * G::kBpb) & ~15LL;
#pragma unroll
      for (int i = 0; i < kPerLane; i++)
        if (lane + 32 * i < 16 * G::kPieces) cp_async16(slot + dst[i], src[i] + base);
      issued++;
    }
    cp_async_commit();
  };
  issue(ring);
  issue(ring + kSlot);
  pdl_launch_dependents();
  if (a.tasks == nullptr) pdl_wait();

  float fin[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) fin[nt][i] = 0.f;
  // chunk 4 G + t of row n sits at x_slot(n, 4 G + t) = n * kStageChunks + 8 (G >> 1) +
  // ((t ^ 4 (n & 1)) ^ (4 (G & 1)) ^ ((G >> 1) & 3)): the lane part is xe, the rest is a constant per G
  const int xe = t ^ ((g & 1) << 2);

  constexpr int kStageCh = kStageK / 256;
  int soff = 0;
  for (int sb = ch0; sb < ch1; sb++) {
    const int rel = sb - ch0;
    if (rel % kStageCh == 0) {
      if (rel != 0) __syncthreads();
      if constexpr (C == IQ2_XXS) {
        stage_x<XT, NT, false>(xs, nullptr, a, s_xrow, tv.m, sb * 256, a.K);
      } else {
        // iq4_xs: lane t of group G multiplies weights 4t+i (low nibbles) and 4t+i+16 (high nibbles),
        // so its chunk holds x[4t], x[4t+16], x[4t+1], x[4t+17], ...
        for (int idx = threadIdx.x; idx < NT * 8 * kStageChunks; idx += kGemvThreads) {
          const int n = idx / kStageChunks, c = idx % kStageChunks;
          const int k = sb * 256 + (c >> 2) * 32 + (c & 3) * 4;
          uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
          if (n < tv.m && k < a.K) {
            const XT* p = static_cast<const XT*>(a.x) + (long long)s_xrow[n] * a.x_row_stride + k;
            if constexpr (sizeof(XT) == 2) {
              lo = __ldg(reinterpret_cast<const uint2*>(p));
              hi = __ldg(reinterpret_cast<const uint2*>(p + 16));
            } else {
              const float4 f0 = __ldg(reinterpret_cast<const float4*>(p));
              const float4 f1 = __ldg(reinterpret_cast<const float4*>(p + 16));
              lo = make_uint2(pack_bf2(f0.x, f0.y), pack_bf2(f0.z, f0.w));
              hi = make_uint2(pack_bf2(f1.x, f1.y), pack_bf2(f1.z, f1.w));
            }
          }
          xs[x_slot(n, c)] = make_uint4(__byte_perm(lo.x, hi.x, 0x5410), __byte_perm(lo.x, hi.x, 0x7632),
                                        __byte_perm(lo.y, hi.y, 0x5410), __byte_perm(lo.y, hi.y, 0x7632));
        }
      }
      __syncthreads();
    }
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncwarp();
    const int ph = (int)(((long long)sb * G::kBpb) & 15);
    const uint8_t* bA = ring + soff + g * G::kStride + ph;
    const uint8_t* bB = ring + soff + (g + 8) * G::kStride + ph;
    const uint4* xsb = xs + (rel % kStageCh) * 32;

    if constexpr (C == IQ4_XS) {
      // [d f16][scales_h u16][scales_l 4 B][qs 128 B]; lane t prepares the scales of groups 2t, 2t+1
      const uint2 hA = *reinterpret_cast<const uint2*>(bA), hB = *reinterpret_cast<const uint2*>(bB);
      float dl[2][2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const uint2 h = r ? hB : hA;
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffff)));
        const uint32_t sh = h.x >> 16, sl = h.y;
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int ib = 2 * t + j;
          const int ls = (int)(((sl >> (4 * ib)) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
          dl[r][j] = d * (float)(ls - 32);
        }
      }
#pragma unroll
      for (int G8 = 0; G8 < 8; G8++) {
        const int from = (lane & ~3) | (G8 >> 1);
        const float dA = __shfl_sync(0xffffffffu, dl[0][G8 & 1], from);
        const float dB = __shfl_sync(0xffffffffu, dl[1][G8 & 1], from);
        const uint32_t WA = *reinterpret_cast<const uint32_t*>(bA + 8 + 16 * G8 + 4 * t);
        const uint32_t WB = *reinterpret_cast<const uint32_t*>(bB + 8 + 16 * G8 + 4 * t);
        uint32_t pa[4], pb[4];
        if constexpr (kHalf) {
          // Two bytes = four nibbles = one permute selector. Entries 0-7 and 8-15 are fetched
          // separately (a selector nibble has 3 index bits), bit 3 of each nibble, spread over its
          // byte by a sign-replicating permute, picks between them. The signed levels then become
          // fp16 exactly: 0x6400 | (v + 128) is 1152 + v.
          auto lut4 = [&](uint32_t X, uint32_t& p0, uint32_t& p1) {
            const uint32_t sel = X & 0x7777u;
            const uint32_t vlo = __byte_perm(T[0], T[1], sel), vhi = __byte_perm(T[2], T[3], sel);
            uint32_t m;  // selector nibbles with bit 3 set replicate the byte's sign bit
            asm("prmt.b32 %0, %1, %2, 0xD9C8;\n" : "=r"(m) : "r"(X << 4), "r"(X));
            uint32_t v;
            asm("lop3.b32 %0, %1, %2, %3, 0xCA;\n" : "=r"(v) : "r"(m), "r"(vhi), "r"(vlo));
            v ^= 0x80808080u;
            const __half2 off = __float2half2_rn(1152.f);
            const uint32_t h0 = __byte_perm(v, 0x64646464u, 0x4140), h1 = __byte_perm(v, 0x64646464u, 0x4342);
            const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&h0), off);
            const __half2 r1 = __hsub2(*reinterpret_cast<const __half2*>(&h1), off);
            p0 = *reinterpret_cast<const uint32_t*>(&r0);
            p1 = *reinterpret_cast<const uint32_t*>(&r1);
          };
          lut4(WA, pa[0], pa[1]);
          lut4(WA >> 16, pa[2], pa[3]);
          lut4(WB, pb[0], pb[1]);
          lut4(WB >> 16, pb[2], pb[3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            pa[i] = tab[(WA >> (8 * i)) & 0xff];
            pb[i] = tab[(WB >> (8 * i)) & 0xff];
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const uint4 xb = xsb[(nt * 8 + g) * kStageChunks + 8 * (G8 >> 1) + (xe ^ ((4 * (G8 & 1)) ^ ((G8 >> 1) & 3)))];
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          if constexpr (kHalf) {
            mma_f16(acc, pa[0], pb[0], pa[1], pb[1], xb.x, xb.y);
            mma_f16(acc, pa[2], pb[2], pa[3], pb[3], xb.z, xb.w);
          } else {
            mma_bf16(acc, pa[0], pb[0], pa[1], pb[1], xb.x, xb.y);
            mma_bf16(acc, pa[2], pb[2], pa[3], pb[3], xb.z, xb.w);
          }
          fin[nt][0] = fmaf(dA, acc[0], fin[nt][0]);
          fin[nt][1] = fmaf(dA, acc[1], fin[nt][1]);
          fin[nt][2] = fmaf(dB, acc[2], fin[nt][2]);
          fin[nt][3] = fmaf(dB, acc[3], fin[nt][3]);
        }
      }
    } else {
      // [d f16][8 x (4 grid-index bytes, u32: 4 x 7-bit sign index + 4-bit scale)], 2-byte aligned
      const float dA0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(bA)));
      const float dB0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(bB)));
      const uint2* grid = reinterpret_cast<const uint2*>(tab);
      // eight lattice bytes -> four pairs of multiplicands (0x6400 | b = 1024 + b in fp16, 0x4300 | b =
      // 128 + b in bf16, minus the offset: exact), signs XOR-ed into the sign bits. The eight sign
      // bits are the 7-bit field plus its parity (ksigns_iq2xs); r carries bit 2j in its low half
      // and bit 2j+1 in its high half once shifted left by 15 - 2j.
      auto make8 = [&](uint2 gb, uint32_t s7, uint4& out) {
        const uint32_t s8 = s7 | ((__popc(s7) & 1u) << 7);
        const uint32_t r = s8 | ((s8 >> 1) << 16);
        const uint32_t magic = kHalf ? 0x64646464u : 0x43434343u;
        uint32_t v[4] = {__byte_perm(gb.x, magic, 0x4140), __byte_perm(gb.x, magic, 0x4342),
                         __byte_perm(gb.y, magic, 0x4140), __byte_perm(gb.y, magic, 0x4342)};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if constexpr (kHalf) {
            const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&v[j]), __float2half2_rn(1024.f));
            v[j] = *reinterpret_cast<const uint32_t*>(&q);
          } else {
            const __nv_bfloat162 q =
                __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v[j]), __float2bfloat162_rn(128.f));
            v[j] = *reinterpret_cast<const uint32_t*>(&q);
          }
          asm("lop3.b32 %0, %1, %2, %3, 0x78;\n" : "=r"(v[j]) : "r"(v[j]), "r"(r << (15 - 2 * j)), "r"(0x80008000u));
        }
        out = make_uint4(v[0], v[1], v[2], v[3]);
      };
#pragma unroll
      for (int G8 = 0; G8 < 8; G8++) {
        const uint8_t* qa = bA + 2 + 8 * G8;
        const uint8_t* qb = bB + 2 + 8 * G8;
        const uint32_t auxA = (uint32_t)*reinterpret_cast<const unsigned short*>(qa + 4) |
                              ((uint32_t)*reinterpret_cast<const unsigned short*>(qa + 6) << 16);
        const uint32_t auxB = (uint32_t)*reinterpret_cast<const unsigned short*>(qb + 4) |
                              ((uint32_t)*reinterpret_cast<const unsigned short*>(qb + 6) << 16);
        const float dA = dA0 * (0.5f + (float)(auxA >> 28)) * 0.25f;
        const float dB = dB0 * (0.5f + (float)(auxB >> 28)) * 0.25f;
        uint4 va, vb;
        make8(grid[qa[t]], (auxA >> (7 * t)) & 127u, va);
        make8(grid[qb[t]], (auxB >> (7 * t)) & 127u, vb);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const uint4 xb = xsb[(nt * 8 + g) * kStageChunks + 8 * (G8 >> 1) + (xe ^ ((4 * (G8 & 1)) ^ ((G8 >> 1) & 3)))];
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          if constexpr (kHalf) {
            mma_f16(acc, va.x, vb.x, va.y, vb.y, xb.x, xb.y);
            mma_f16(acc, va.z, vb.z, va.w, vb.w, xb.z, xb.w);
          } else {
            mma_bf16(acc, va.x, vb.x, va.y, vb.y, xb.x, xb.y);
            mma_bf16(acc, va.z, vb.z, va.w, vb.w, xb.z, xb.w);
          }
          fin[nt][0] = fmaf(dA, acc[0], fin[nt][0]);
          fin[nt][1] = fmaf(dA, acc[1], fin[nt][1]);
          fin[nt][2] = fmaf(dB, acc[2], fin[nt][2]);
          fin[nt][3] = fmaf(dB, acc[3], fin[nt][3]);
        }
      }
    }
    __syncwarp();  // the slot is free again
    issue(ring + soff);
    soff ^= kSlot;
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  // ---- partial tile -> shared memory -> cluster reduce (as in gemv_kernel)
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int tok = nt * 8 + 2 * t + (i & 1);
      const int row = warp * 16 + g + 8 * (i >> 1);
      red[tok * kRowsPerCta + row] = fin[nt][i];
    }
  cluster.sync();
  const float* peer[kMaxSplit];
#pragma unroll
  for (int s = 0; s < kMaxSplit; s++) peer[s] = s < S ? cluster.map_shared_rank(red, s) : red;
  const int cta_row0 = blockIdx.x * kRowsPerCta;
  for (int idx = slice + S * threadIdx.x; idx < kTile; idx += S * kGemvThreads) {
    const int tok = idx / kRowsPerCta, row = idx % kRowsPerCta;
    if (tok < tv.m && cta_row0 + row < a.N) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxSplit; s++)
        if (s < S) sum += peer[s][idx];
      MT* y = static_cast<MT*>(a.y) + (long long)s_yrow[tok] * a.y_row_stride + cta_row0 + row;
      if constexpr (kHalf) *y = __float2half_rn(sum);
      else *y = __float2bfloat16_rn(sum);
    }
  }
  cluster_sync_relaxed();
}

template <int C, typename XT, int NT>
static cudaError_t launch_iq(const GemvArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = gemv_iq_kernel<C, XT, NT>;
  constexpr int dyn = kGemvWarps * kRing * 16 * IqGeom<C>::kStride;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = grid.y;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.tasks == nullptr ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int C>
static cudaError_t launch_iq_any(int x_dtype, const GemvArgs& a, dim3 grid, bool nt2, cudaStream_t st) {
  if (x_dtype == F16) return nt2 ? launch_iq<C, __half, 2>(a, grid, st) : launch_iq<C, __half, 1>(a, grid, st);
  if (x_dtype == BF16)
    return nt2 ? launch_iq<C, __nv_bfloat16, 2>(a, grid, st) : launch_iq<C, __nv_bfloat16, 1>(a, grid, st);
  return nt2 ? launch_iq<C, float, 2>(a, grid, st) : launch_iq<C, float, 1>(a, grid, st);
}

// ------------------------------------------------------------------ launch
template <int C, int A, typename XT, int NT, bool FAST>
static cudaError_t launch_k(const GemvArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = gemv_kernel<C, A, XT, NT, FAST>;
  const size_t dyn = FAST ? (size_t)kRingBytesPerCta : 0;
  if (dyn > 0) {
    static bool attr_set[16] = {};  // per device, set once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
      if (e != cudaSuccess) return e;
      attr_set[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = grid.y;
  attr[0].val.clusterDim.z = 1;
  // dense calls overlap their weight prefetch with the tail of the previous kernel
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.tasks == nullptr ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, a);
}

static cudaError_t launch_m1(const GemvArgs& a, dim3 grid, cudaStream_t st) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_m1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kRingBytesPerCta);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = kRingBytesPerCta;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = grid.y;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 1 : 2;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_m1_kernel, a);
}

static cudaError_t launch_m1_rows(const GemvArgs& a, cudaStream_t st) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_m1_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         rows_dyn_smem(kRowsMaxK));
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + 15) / 16, 1, 1);
  cfg.blockDim = dim3(kRowsThreads);
  cfg.dynamicSmemBytes = rows_dyn_smem(a.K);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_m1_rows_kernel, a);
}

template <typename XT>
static cudaError_t launch_m1_dp4a(const GemvArgs& a, cudaStream_t st) {
  const int nchunks = a.K >> 8;
  const int per = (nchunks + kDpWarps - 1) / kDpWarps;
  const int D = per < 2 ? 1 : 2;  // 74 KB of ring: two CTAs per SM
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q4k_m1_dp4a_kernel<XT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         dp_dyn_smem(kDpMaxK, 2));
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  // fewer than one 32-row CTA per SM: spread the rows over all 148 SMs instead (28 rows each for N = 4096)
  int rpc = kDpRows;
  if ((a.N + kDpRows - 1) / kDpRows < 148 && a.N >= 148 * 16) rpc = (a.N + 147) / 148;
  cfg.gridDim = dim3((a.N + rpc - 1) / rpc, 1, 1);
  cfg.blockDim = dim3(kDpThreads);
  cfg.dynamicSmemBytes = dp_dyn_smem(a.K, D);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("KQ_NO_PDL") != nullptr;  // A/B lever
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, gemv_q4k_m1_dp4a_kernel<XT>, a, D, rpc);
}

template <int C, int NAT>
static cudaError_t launch_generic(int x_dtype, const GemvArgs& a, dim3 grid, bool nt2, bool aligned, cudaStream_t st) {
#define KQ_GV(AL, XT) \
  return nt2 ? launch_k<C, AL, XT, 2, false>(a, grid, st) : launch_k<C, AL, XT, 1, false>(a, grid, st)
  if (aligned) {
    if (x_dtype == F16) KQ_GV(NAT, __half);
    if (x_dtype == BF16) KQ_GV(NAT, __nv_bfloat16);
    KQ_GV(NAT, float);
  } else {
    if (x_dtype == F16) KQ_GV(1, __half);
    if (x_dtype == BF16) KQ_GV(1, __nv_bfloat16);
    KQ_GV(1, float);
  }
#undef KQ_GV
}

cudaError_t launch_gemv(int codec, int x_dtype, const GemvArgs& a, cudaStream_t st) {
  if (a.N <= 0 || a.K <= 0) return cudaSuccess;
  const int groups = a.tasks ? a.n_tasks : (a.M + 15) / 16;
  if (groups <= 0) return cudaSuccess;
  if (groups > 65535) return cudaErrorInvalidConfiguration;
  // K split (= cluster size). Measured on B200: what matters is (a) at least two
  // CTAs per SM, whatever it costs, and (b) beyond that, slices of at least four
  // 256-weight chunks so that the per-CTA prologue and cluster reduce amortise.
  const int row_groups = (a.N + kRowsPerCta - 1) / kRowsPerCta;
  const int nchunks = (a.K + 255) / 256;
  int S = 1;
  while (S < kMaxSplit && S * 2 <= nchunks) {
    const long long ctas = (long long)row_groups * groups * S;
    if (ctas >= 4 * 148) break;
    if (ctas >= 2 * 148 && nchunks / (2 * S) < 4) break;
    S *= 2;
  }
  // A/B lever: KQ_GEMV_SPLIT=1|2|4|8 overrides the K-split heuristic.
  static const char* const split_env = std::getenv("KQ_GEMV_SPLIT");  // read once per process
  if (const char* env = split_env) {
    const int v = std::atoi(env);
    if ((v == 1 || v == 2 || v == 4 || v == 8) && v <= nchunks) S = v;
  }
  const dim3 grid(row_groups, S, groups);
  const bool nt2 = a.tasks ? (a.max_m > 8) : (a.M > 8);
  const bool aligned = a.w_align16 != 0;

  // A/B lever: KQ_GEMV_IMMA=0|1, the integer tensor-pipe kernel for one or two dense rows of q4_k
  // (measured against the kernels below: 3-7 % faster up to ~60 M weights, slower beyond)
  static const char* imma_env = std::getenv("KQ_GEMV_IMMA");
  static const char* int_env = std::getenv("KQ_GEMV_DP4A");  // = 0 switches every integer kernel off
  const bool imma_on = imma_env ? imma_env[0] == '1'
                                : (!(int_env && int_env[0] == '0') && (long long)a.N * a.K <= (60ll << 20));
  // A/B lever: KQ_GEMV_STREAM=0 keeps one-wave matrices on the kernels below
  static const bool stream_on = [] {
    const char* e = std::getenv("KQ_GEMV_STREAM");
    return !(e && e[0] == '0');
  }();
  if (stream_on && !(int_env && int_env[0] == '0') && gemv_stream_supported(codec, x_dtype, a))
    return launch_gemv_stream(x_dtype, a, st);
  if (imma_on && gemv_imma_supported(codec, x_dtype, a)) return launch_gemv_imma(x_dtype, a, st);
  // one dense activation row of q4_k: the integer dot-product kernel. A/B lever: KQ_GEMV_DP4A=0|1.
  // Measured: it wins up to ~60 M weights against the fp16 tensor-core kernels below (which win
  // beyond), and always against the generic path that bf16 / float activations would take.
  static const char* dp_env = std::getenv("KQ_GEMV_DP4A");
  const bool dp_on = dp_env ? dp_env[0] == '1' : (x_dtype != F16 || (long long)a.N * a.K <= (60ll << 20));
  if (dp_on && codec == Q4_K && aligned && a.tasks == nullptr && a.M == 1 && (a.K & 255) == 0 && a.K <= kDpMaxK &&
      (a.row_bytes & 15) == 0) {
    if (x_dtype == F16) return launch_m1_dp4a<__half>(a, st);
    if (x_dtype == BF16) return launch_m1_dp4a<__nv_bfloat16>(a, st);
    return launch_m1_dp4a<float>(a, st);
  }
  // KQ_GEMV_DP4A=0 also switches the other codecs' integer kernels off
  if (!(dp_env && dp_env[0] == '0') && gemv_dp4a_supported(codec, x_dtype, a)) return launch_gemv_dp4a(codec, x_dtype, a, st);
  static const bool no_m1 = std::getenv("KQ_GEMV_NO_M1") != nullptr;  // A/B lever
  if (codec == Q4_K && x_dtype == F16 && aligned && a.tasks == nullptr && a.M == 1 && !no_m1) {
    // The cluster-free kernel wins (measured) unless few row groups leave each warp a long K
    // chain. A/B lever: KQ_GEMV_ROWS=0|1 forces the choice.
    static const char* rows_env = std::getenv("KQ_GEMV_ROWS");
    const int row_ctas = (a.N + 15) / 16;
    const int sb_per_warp = (nchunks + kRowsWarps - 1) / kRowsWarps;
    bool rows = a.K <= kRowsMaxK && ((row_ctas >= 148 && sb_per_warp <= 4) || row_ctas >= 3 * 148);
    if (rows_env) rows = rows_env[0] == '1' && a.K <= kRowsMaxK && row_ctas <= 65535;
    if (rows) return launch_m1_rows(a, st);
    return launch_m1(a, grid, st);
  }
  // rows that are whole numbers of 16 bytes let the ring copy aligned windows around each block
  static const bool no_iq = std::getenv("KQ_GEMV_NO_IQ") != nullptr;  // A/B lever
  if (aligned && (a.row_bytes & 15) == 0 && !no_iq) {
    if (codec == IQ4_XS) return launch_iq_any<IQ4_XS>(x_dtype, a, grid, nt2, st);
    if (codec == IQ2_XXS) return launch_iq_any<IQ2_XXS>(x_dtype, a, grid, nt2, st);
  }
  if (codec == Q4_K && x_dtype == F16 && aligned)
    return nt2 ? launch_k<Q4_K, 16, __half, 2, true>(a, grid, st) : launch_k<Q4_K, 16, __half, 1, true>(a, grid, st);
  switch (codec) {
    case Q2_K: return launch_generic<Q2_K, 4>(x_dtype, a, grid, nt2, aligned, st);
    case Q3_K: return launch_generic<Q3_K, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q4_K: return launch_generic<Q4_K, 16>(x_dtype, a, grid, nt2, aligned, st);
    case Q5_K: return launch_generic<Q5_K, 16>(x_dtype, a, grid, nt2, aligned, st);
    case Q6_K: return launch_generic<Q6_K, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q4_0: return launch_generic<Q4_0, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q8_0: return launch_generic<Q8_0, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ4_NL: return launch_generic<IQ4_NL, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ4_XS: return launch_generic<IQ4_XS, 8>(x_dtype, a, grid, nt2, aligned, st);
    case IQ2_XXS: return launch_generic<IQ2_XXS, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q4_1: return launch_generic<Q4_1, 4>(x_dtype, a, grid, nt2, aligned, st);
    case Q5_0: return launch_generic<Q5_0, 2>(x_dtype, a, grid, nt2, aligned, st);
    case Q5_1: return launch_generic<Q5_1, 8>(x_dtype, a, grid, nt2, aligned, st);
    case IQ3_XXS: return launch_generic<IQ3_XXS, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ3_S: return launch_generic<IQ3_S, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ2_XS: return launch_generic<IQ2_XS, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ2_S: return launch_generic<IQ2_S, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ1_S: return launch_generic<IQ1_S, 2>(x_dtype, a, grid, nt2, aligned, st);
    case IQ1_M: return launch_generic<IQ1_M, 8>(x_dtype, a, grid, nt2, aligned, st);
    case MXFP4: return launch_generic<MXFP4, 1>(x_dtype, a, grid, nt2, aligned, st);
    case NVFP4: return launch_generic<NVFP4, 4>(x_dtype, a, grid, nt2, aligned, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace kq
