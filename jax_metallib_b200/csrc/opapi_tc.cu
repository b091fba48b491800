// Affine 4- and 8-bit matmuls of the operator API at decode sizes (f16 activations, M <= 16) on the
// tensor cores, fed by TMA.
//
//   y[m,n] = sum_g ( s[n,g] * sum_{k in g} x[m,k] q[n,k]  +  b[n,g] * sum_{k in g} x[m,k] )
//
// The packed words go to mma.sync.m16n8k16 as they are: an AND leaves two codes of a word in the low
// bits of the two halves of a register, where each reads as the f16 subnormal q * 2^-24 (exact; the
// factor 2^24 multiplies the result once at the end).  A 4-bit code may also stay at bits 4-7, where
// it is worth 16 q * 2^-24: those products go to a second accumulator that is added with weight 1/16,
// which saves the shifts that would bring every code down to bit 0 and scales no activation.  The 16
// rows of the MMA's first operand are 16 output columns, the 16 k-slots of one MMA are four codes of
// one packed word per thread of a quad, and the activations are staged in shared memory once per CTA
// in that slot order, so that a thread's fragments are plain 8- and 16-byte shared loads.
//
// Work split: a CTA owns `tiles` 16-column tiles, each cut `ksplit` ways along K; one warp per (tile,
// K part), partial sums combined through shared memory in a fixed order.  Every warp runs its own
// ring of TMA boxes (16 rows x 128 bytes of packed weights, 128-byte swizzle) on its own mbarriers,
// and fetches the scales and biases of its rows and groups with two more boxes, so no warp waits for
// another inside the main loop.  The first boxes are requested before the activations are staged.
//
// Per 64 weights of a row the main loop issues 1 shared load of weights, 2 of activations (4-bit), 10
// logic instructions, 2 MMAs and, per group, 12 FMAs; that is what bounds it, not the MMA rate.
#include <atomic>

#include "common.cuh"

namespace qmm {
namespace opapi_tc {

constexpr int kMaxWarps = 16;
constexpr int kBox = 2048;           // one TMA box: 16 rows x 128 bytes
constexpr int kStepBytes = 32;       // bytes of a weight row per step of a quad: 4 threads x 8 bytes
constexpr int kStepsPerChunk = 4;    // a box holds 4 steps
constexpr int kGroupsPerBox = 32;    // scales / biases of 32 groups per row in one box
constexpr int kMaxSmem = 227 * 1024;

namespace dev {
using namespace qmm::dev;

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same with a zero accumulator coming in: the first MMA of a group
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("{\n\t.reg .f32 z;\n\tmov.f32 z, 0f00000000;\n\t"
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {z, z, z, z};\n\t}"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// shared loads by 32-bit address with a compile-time offset (folds into the instruction)
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
  return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
template <int OFF>
__device__ __forceinline__ float2 lds64f(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(a), "n"(OFF));
  return v;
}
// Warp-wide bounded wait for a box: one try (the usual case once the ring is primed), then the sleeping wait.
// All lanes leave with the same answer.
__device__ __forceinline__ bool wait_box(uint64_t* bar, uint32_t parity, int* status, int tag) {
  if (__all_sync(0xFFFFFFFFu, mbar_try_wait(bar, parity))) return true;
  return mbar_wait_relaxed_warp(bar, parity, status, tag);
}
__device__ __forceinline__ float sel4(const float4& v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); }
}  // namespace dev

template <int BITS>
struct Fmt {
  static constexpr int kStepK = kStepBytes * 8 / BITS;   // k per step: 64 (4-bit) or 32 (8-bit)
  static constexpr int kXStep = kStepK * 2;              // bytes of a staged activation row per step
  // staged rows are padded so that the rows of a quarter-warp's 16-byte loads fall into different banks:
  // a quad reads 4 x 16 bytes 32 apart (4-bit) or 64 contiguous bytes (8-bit)
  static constexpr int kRowPad = BITS == 4 ? 16 : 64;
};

struct Plan {
  int tiles, ksplit, stages, warps;
  unsigned grid;
  size_t smem;
};

// Shared memory of one CTA, in this order (the first two are 1024-byte aligned for the swizzle):
//   weight rings [warps][stages][2048] | scale and bias boxes [warps][2][2048] | activations [M][2K + pad] |
//   group sums [G][8 MT] f32 | hand-over [warps][32][4 MT] f32 | mbarriers [warps][stages + 1]
static size_t fixed_smem(int bits, int warps, int M, int MT, int K, int G) {
  const int pad = bits == 4 ? Fmt<4>::kRowPad : Fmt<8>::kRowPad;
  return static_cast<size_t>(warps) * 2 * kBox + static_cast<size_t>(M) * (2 * K + pad) + static_cast<size_t>(G) * MT * 8 * 4 +
         static_cast<size_t>(warps) * 32 * MT * 4 * 4 + static_cast<size_t>(warps) * (8 + 1) * 8 + 1024;
}

// How to cut the problem; false when this kernel does not cover it.
static bool plan(int bits, int64_t M, int64_t N, int64_t K, int64_t gs, Plan* p) {
  const int step_k = bits == 4 ? Fmt<4>::kStepK : Fmt<8>::kStepK;
  const int64_t spg = gs / step_k;                       // steps per group
  if (gs % step_k != 0 || (spg != 1 && spg != 2 && spg != 4)) return false;
  if (N % 16 != 0 || K % gs != 0 || K * bits / 8 < 128 || K > (1 << 17)) return false;
  const int64_t G = K / gs;
  if (G % 4 != 0) return false;                          // K parts begin on 4 groups: 16 bytes of a scale row, one box of weights
  const int U = static_cast<int>(G / 4);
  const int ksplit_min = (U + 7) / 8;                    // at most 32 groups per warp: one box of scales
  if (ksplit_min > kMaxWarps) return false;
  const int64_t tiles_total = N / 16;
  const int sms = num_sms();
  int tiles = static_cast<int>((tiles_total + sms - 1) / sms);
  if (tiles * ksplit_min > kMaxWarps) tiles = kMaxWarps / ksplit_min;
  int ksplit = kMaxWarps / tiles;
  if (ksplit > U) ksplit = U;
  p->tiles = tiles;
  p->ksplit = ksplit;
  p->warps = tiles * ksplit;
  p->grid = static_cast<unsigned>((tiles_total + tiles - 1) / tiles);
  const int MT = M <= 8 ? 1 : 2;
  const size_t fixed = fixed_smem(bits, p->warps, static_cast<int>(M), MT, static_cast<int>(K), static_cast<int>(G));
  if (fixed + static_cast<size_t>(p->warps) * 2 * kBox > static_cast<size_t>(kMaxSmem)) return false;
  const int chunks_per_warp = static_cast<int>((((U + ksplit - 1) / ksplit) * 4 * spg + kStepsPerChunk - 1) / kStepsPerChunk);
  int stages = static_cast<int>((kMaxSmem - fixed) / (static_cast<size_t>(p->warps) * kBox));
  if (stages > 8) stages = 8;
  if (stages > chunks_per_warp) stages = chunks_per_warp;
  if (stages < 1) return false;
  p->stages = stages;
  p->smem = fixed + static_cast<size_t>(p->warps) * stages * kBox;
  return true;
}

template <int BITS, int MT, int SPG>
__global__ void __launch_bounds__(kMaxWarps * 32)
affine_ring_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                   const __grid_constant__ CUtensorMap bmap, const __half* __restrict__ x, __half* __restrict__ y, int M,
                   int N, int K, int gs, int stages, int tiles, int ksplit, int* status) {
  using namespace dev;
  using F = Fmt<BITS>;
  constexpr int GPC = kStepsPerChunk / SPG;                 // groups per chunk: 4, 2 or 1
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // the swizzle pattern repeats every 1024 bytes
  const int threads = blockDim.x, warps = threads >> 5;
  const int G = K / gs;
  const int row_bytes = K * 2 + F::kRowPad;
  uint8_t* ring = smem;
  uint8_t* sbox = ring + warps * stages * kBox;
  uint8_t* xs = sbox + warps * 2 * kBox;
  float* xsum = reinterpret_cast<float*>(xs + M * row_bytes);
  float* hand = xsum + G * MT * 8;
  uint64_t* bars = reinterpret_cast<uint64_t*>(hand + warps * 32 * MT * 4);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = warp % tiles, ks = warp / tiles;
  const int n0 = (blockIdx.x * tiles + tile) * 16;
  const int g8 = lane >> 2, t4 = lane & 3;
  // A thread's two rows of a box are rho and rho + 8: with the 128-byte swizzle the four rows that one
  // phase of an 8-byte shared load touches then sit in four different pairs of 16-byte chunks.
  const int rho = ((g8 & 3) << 1) | (g8 >> 2);
  const bool active = n0 < N;
  const int U = G >> 2;
  const int g_begin = ((U * ks) / ksplit) << 2, g_end = ((U * (ks + 1)) / ksplit) << 2;
  const int total = active ? (g_end - g_begin) * SPG : 0;   // steps; a multiple of 4
  const int nchunks = total / kStepsPerChunk;
  const int seg_begin = g_begin * (gs * BITS / 8);           // byte offset of this warp's K part within a row
  uint8_t* my_ring = ring + warp * stages * kBox;
  uint8_t* my_sbox = sbox + warp * 2 * kBox;
  uint64_t* my_bar = bars + warp * (stages + 1);             // [stages] = the scale and bias boxes

  if (lane == 0) {
    for (int i = 0; i <= stages; ++i) mbar_init(my_bar + i, 1);
    fence_mbar_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  pdl_wait();                 // everything below may read what the previous kernel wrote
  pdl_launch_dependents();
  if (lane == 0) {
    if (active) {
      mbar_expect_tx(my_bar + stages, 2 * kBox);
      tma_load_2d(my_sbox, &smap, my_bar + stages, g_begin, n0);
      tma_load_2d(my_sbox + kBox, &bmap, my_bar + stages, g_begin, n0);
      for (int c = 0; c < stages && c < nchunks; ++c) {
        mbar_expect_tx(my_bar + c, kBox);
        tma_load_2d(my_ring + c * kBox, &wmap, my_bar + c, seg_begin + c * 128, n0);
      }
    }
  }
  __syncwarp();

  // ---- activations: 8 k (16 bytes) per thread and pass, stored in MMA slot order; sums per (row, group)
  //   4-bit: (x0,x4) (x2,x6) | (x1,x5) (x3,x7)     one packed word; the second pair meets the codes at bits 4-7
  //   8-bit: (x0,x2) (x1,x3) | (x4,x6) (x5,x7)     two packed words
  const int chunks = K / 8;
  const int lanes_per_group = gs / 8;
  const bool fused_sum = lanes_per_group <= 32 && (lanes_per_group & (lanes_per_group - 1)) == 0;
  {
    const int n_it = M * chunks;
    int m = 0, c8 = tid;                                    // i = m * chunks + c8, advanced without a division
    while (c8 >= chunks) { c8 -= chunks; ++m; }
    for (int i0 = tid; i0 - tid < n_it; i0 += threads * 4) {   // whole warps stay in the loop for the shuffles
      uint4 v[4];
      int mm[4], cc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j * threads;
        mm[j] = m;
        cc[j] = c8;
        v[j] = i < n_it ? __ldg(reinterpret_cast<const uint4*>(x) + i) : make_uint4(0, 0, 0, 0);
        c8 += threads;
        while (c8 >= chunks) { c8 -= chunks; ++m; }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j * threads;
        if (i - lane >= n_it) continue;                     // warp-uniform
        const uint32_t h0 = v[j].x, h1 = v[j].y, h2 = v[j].z, h3 = v[j].w;   // (x0,x1) (x2,x3) (x4,x5) (x6,x7)
        if (i < n_it) {
          uint4 o;
          if (BITS == 4) {
            o.x = __byte_perm(h0, h2, 0x5410);
            o.y = __byte_perm(h1, h3, 0x5410);
            o.z = __byte_perm(h0, h2, 0x7632);
            o.w = __byte_perm(h1, h3, 0x7632);
          } else {
            o.x = __byte_perm(h0, h1, 0x5410);
            o.y = __byte_perm(h0, h1, 0x7632);
            o.z = __byte_perm(h2, h3, 0x5410);
            o.w = __byte_perm(h2, h3, 0x7632);
          }
          *reinterpret_cast<uint4*>(xs + mm[j] * row_bytes + cc[j] * 16) = o;
        }
        if (fused_sum) {
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
          const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&h2));
          const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&h3));
          float p = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
          for (int o = 1; o < lanes_per_group; o <<= 1) p += __shfl_xor_sync(0xFFFFFFFFu, p, o);
          if (i < n_it && (cc[j] & (lanes_per_group - 1)) == 0) xsum[(cc[j] / lanes_per_group) * (MT * 8) + mm[j]] = p;
        }
      }
    }
  }
  // rows m >= M only feed result columns that are never stored; keep them finite
  for (int i = tid; i < G * MT * 8; i += threads)
    if ((i % (MT * 8)) >= M) xsum[i] = 0.f;
  __syncthreads();
  if (!fused_sum) {
    for (int i = tid; i < M * G; i += threads) {
      const int g = i / M, m = i - g * M;
      float acc = 0.f;
      const uint8_t* src = xs + m * row_bytes + g * gs * 2;
      for (int k = 0; k < gs * 2; k += 16) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + k);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
        acc += ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
      }
      xsum[g * (MT * 8) + m] = acc;
    }
    __syncthreads();
  }

  // ---- main loop: one warp, its own ring
  float ys[MT][4], yb[MT][4];      // sum of s * (x . q) 2^-24 and of b * sum(x), kept apart so that 2^24 multiplies once
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) ys[mt][i] = yb[mt][i] = 0.f;
  bool ok = true;
  int consumed = 0, requested = stages < nchunks ? stages : nchunks;
  if (active) {
    // byte offset of this thread's 8 bytes of step 0 within a box: row rho, 16-byte chunk (t4 >> 1) ^ rho
    const uint32_t wthread = rho * 128 + (((t4 >> 1) ^ rho) << 4) + ((t4 & 1) << 3);
    // rows m >= M read row M - 1: their products land in result columns that are not stored
    uint32_t xa[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int row = min(mt * 8 + g8, M - 1);
      xa[mt] = smem_u32(xs) + row * row_bytes + (g_begin * (gs / 8) + (BITS == 4 ? 2 * t4 : t4)) * 16;
    }
    // scales of rows rho and rho + 8 (+ 1024), biases one box further: 4 groups per 16-byte chunk, chunk j at j ^ rho
    const uint32_t sa = smem_u32(my_sbox) + rho * 128;
    uint32_t xsa = smem_u32(xsum) + (g_begin * MT * 8 + 2 * t4) * 4;
    ok = wait_box(my_bar + stages, 0, status, 70);
    constexpr uint32_t kLo4 = 0x000F000Fu, kHi4 = 0x00F000F0u, kByte = 0x00FF00FFu;
    float d1[MT][4], d16[MT][4];
    int st = 0, prev_st = 0, gq = 0;
    uint32_t phase = 0;
    const uint32_t ring32 = smem_u32(my_ring);
    for (int c = 0; c < nchunks && ok; ++c) {
      ok = wait_box(my_bar + st, phase, status, 71);
      if (!ok) break;
      if (c >= 1 && requested < nchunks) {      // refill the box that the previous iteration has finished reading
        if (lane == 0) {
          mbar_expect_tx(my_bar + prev_st, kBox);
          tma_load_2d(my_ring + prev_st * kBox, &wmap, my_bar + prev_st, seg_begin + requested * 128, n0);
        }
        ++requested;
      }
      // this chunk's GPC groups: chunk gq >> 2 of the scale rows, components (gq & 3) ..
      const uint32_t sq = sa + ((((gq >> 2) ^ rho) & 7) << 4);
      const float4 s_lo = lds128f(sq), s_hi = lds128f(sq + 1024), b_lo = lds128f(sq + kBox), b_hi = lds128f(sq + kBox + 1024);
      const uint32_t wbase = (ring32 + st * kBox) | wthread;
#pragma unroll
      for (int s4 = 0; s4 < kStepsPerChunk; ++s4) {
        const uint32_t wa = wbase ^ (s4 << 5);
        const uint2 a = lds64<0>(wa), b = lds64<1024>(wa);
        const bool first = s4 % SPG == 0;
        if (BITS == 4) {
#pragma unroll
          for (int wi = 0; wi < 2; ++wi) {
            const uint32_t lo = wi ? a.y : a.x, hi = wi ? b.y : b.x;
            const uint32_t lo8 = lo >> 8, hi8 = hi >> 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xq = wi ? (s4 == 0 ? lds128<16>(xa[mt]) : s4 == 1 ? lds128<128 + 16>(xa[mt]) : s4 == 2 ? lds128<256 + 16>(xa[mt]) : lds128<384 + 16>(xa[mt]))
                                  : (s4 == 0 ? lds128<0>(xa[mt]) : s4 == 1 ? lds128<128>(xa[mt]) : s4 == 2 ? lds128<256>(xa[mt]) : lds128<384>(xa[mt]));
              if (wi == 0 && first) {
                mma16816_first(d1[mt], lo & kLo4, hi & kLo4, lo8 & kLo4, hi8 & kLo4, xq.x, xq.y);
                mma16816_first(d16[mt], lo & kHi4, hi & kHi4, lo8 & kHi4, hi8 & kHi4, xq.z, xq.w);
              } else {
                mma16816(d1[mt], lo & kLo4, hi & kLo4, lo8 & kLo4, hi8 & kLo4, xq.x, xq.y);
                mma16816(d16[mt], lo & kHi4, hi & kHi4, lo8 & kHi4, hi8 & kHi4, xq.z, xq.w);
              }
            }
          }
        } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xq = s4 == 0 ? lds128<0>(xa[mt]) : s4 == 1 ? lds128<64>(xa[mt]) : s4 == 2 ? lds128<128>(xa[mt]) : lds128<192>(xa[mt]);
            if (first) mma16816_first(d1[mt], a.x & kByte, b.x & kByte, (a.x >> 8) & kByte, (b.x >> 8) & kByte, xq.x, xq.y);
            else mma16816(d1[mt], a.x & kByte, b.x & kByte, (a.x >> 8) & kByte, (b.x >> 8) & kByte, xq.x, xq.y);
            mma16816(d1[mt], a.y & kByte, b.y & kByte, (a.y >> 8) & kByte, (b.y >> 8) & kByte, xq.z, xq.w);
          }
        }
        if (s4 % SPG == SPG - 1) {      // a group ends
          const int j = (GPC == 4) ? s4 : ((gq & 3) + s4 / SPG);   // component of the 4-group chunk; static when GPC == 4
          const float sl = sel4(s_lo, j & 3), sh = sel4(s_hi, j & 3), bl = sel4(b_lo, j & 3), bh = sel4(b_hi, j & 3);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float2 xv = s4 / SPG == 0 ? lds64f<0>(xsa + mt * 32) : s4 / SPG == 1 ? lds64f<MT * 32>(xsa + mt * 32)
                              : s4 / SPG == 2 ? lds64f<2 * MT * 32>(xsa + mt * 32) : lds64f<3 * MT * 32>(xsa + mt * 32);
            float t0 = d1[mt][0], t1 = d1[mt][1], t2 = d1[mt][2], t3 = d1[mt][3];
            if (BITS == 4) {
              t0 = fmaf(d16[mt][0], 0.0625f, t0);
              t1 = fmaf(d16[mt][1], 0.0625f, t1);
              t2 = fmaf(d16[mt][2], 0.0625f, t2);
              t3 = fmaf(d16[mt][3], 0.0625f, t3);
            }
            ys[mt][0] = fmaf(sl, t0, ys[mt][0]);
            ys[mt][1] = fmaf(sl, t1, ys[mt][1]);
            ys[mt][2] = fmaf(sh, t2, ys[mt][2]);
            ys[mt][3] = fmaf(sh, t3, ys[mt][3]);
            yb[mt][0] = fmaf(bl, xv.x, yb[mt][0]);
            yb[mt][1] = fmaf(bl, xv.y, yb[mt][1]);
            yb[mt][2] = fmaf(bh, xv.x, yb[mt][2]);
            yb[mt][3] = fmaf(bh, xv.y, yb[mt][3]);
          }
        }
      }
      gq += GPC;
      xsa += GPC * MT * 32;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xa[mt] += kStepsPerChunk * F::kXStep;
      __syncwarp();
      ++consumed;
      prev_st = st;
      if (++st == stages) { st = 0; phase ^= 1; }
    }
    if (!ok) {
      // a wait gave up (recorded in the status word): let the boxes still in flight land, each wait bounded
      // again, so that nothing writes into this CTA's shared memory after it has gone
      for (int c = consumed + 1; c < requested; ++c) {
        if (++st == stages) { st = 0; phase ^= 1; }
        mbar_wait_relaxed_warp(my_bar + st, phase, nullptr, 0);
      }
    }
  }
  // ---- K parts meet in shared memory; part 0 adds them in order and stores
  float* slot = hand + (warp * 32 + lane) * MT * 4;
  if (ks != 0 && active) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) slot[mt * 4 + i] = fmaf(ys[mt][i], 16777216.f, yb[mt][i]);
  }
  __syncthreads();
  if (ks == 0 && active) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = fmaf(ys[mt][i], 16777216.f, yb[mt][i]);
        for (int o = 1; o < ksplit; ++o) v += hand[((o * tiles + tile) * 32 + lane) * MT * 4 + mt * 4 + i];
        const int n = n0 + rho + ((i >> 1) << 3), m = mt * 8 + 2 * t4 + (i & 1);
        if (m < M) y[static_cast<size_t>(m) * N + n] = __float2half_rn(v);
      }
    }
  }
}

template <int BITS, int MT, int SPG>
static int launch_one(const Plan& p, const CUtensorMap& wmap, const CUtensorMap& smap, const CUtensorMap& bmap, const void* x,
                      void* y, int M, int N, int K, int gs, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};
  auto kernel = affine_ring_kernel<BITS, MT, SPG>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxSmem, configured)) return rc;
  cudaError_t e = launch_pdl(kernel, dim3(p.grid), dim3(p.warps * 32), p.smem, stream, wmap, smap, bmap,
                             static_cast<const __half*>(x), static_cast<__half*>(y), M, N, K, gs, p.stages, p.tiles, p.ksplit,
                             device_status_word());
  if (e != cudaSuccess)
    return set_error(QMM_ERR_CUDA, "affine_qgemm_%dbit_f16 (TMA ring): launch failed: %s", BITS, cudaGetErrorString(e));
  return QMM_OK;
}

template <int BITS>
static int launch_bits(const Plan& p, const CUtensorMap& wmap, const CUtensorMap& smap, const CUtensorMap& bmap, const void* x,
                       void* y, int M, int N, int K, int gs, cudaStream_t stream) {
  const int spg = gs / Fmt<BITS>::kStepK;
  if (M <= 8) {
    if (spg == 1) return launch_one<BITS, 1, 1>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
    if (spg == 2) return launch_one<BITS, 1, 2>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
    return launch_one<BITS, 1, 4>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
  }
  if (spg == 1) return launch_one<BITS, 2, 1>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
  if (spg == 2) return launch_one<BITS, 2, 2>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
  return launch_one<BITS, 2, 4>(p, wmap, smap, bmap, x, y, M, N, K, gs, stream);
}

}  // namespace opapi_tc

// True when the TMA-ring kernel covers the call (f16 activations, 1 <= M <= 16, groups of 1, 2 or 4 steps
// of a quad, a multiple of 4 groups per row, 16-byte aligned operands, shared memory for at least one box
// per warp beside the staged activations).
bool affine_ring_covers(int64_t M, int64_t N, int64_t K, int bits, int64_t gs, int dtype, const void* x, const void* w,
                        const float* scales, const float* biases) {
  using namespace opapi_tc;
  if ((bits != 4 && bits != 8) || dtype != QMM_F16 || M < 1 || M > 16) return false;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(scales, 16) || !aligned(biases, 16)) return false;
  Plan p;
  return plan(bits, M, N, K, gs, &p);
}

int affine_ring_launch(int bits, const void* x, const void* w, const float* scales, const float* biases, void* y, int64_t M,
                       int64_t N, int64_t K, int64_t gs, void* stream) {
  using namespace opapi_tc;
  Plan p;
  QMM_REQUIRE(plan(bits, M, N, K, gs, &p), QMM_ERR_UNSUPPORTED, "affine_ring_launch: shape not covered");
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "qmm_affine_matmul: an earlier kernel gave up a wait (status 0x%x); "
                     "call qmm_clear_device_status() after handling it", st);
  CUtensorMap wmap, smap, bmap;
  const uint64_t row_bytes = static_cast<uint64_t>(K) * bits / 8;
  const uint64_t G = static_cast<uint64_t>(K / gs);
  if (int rc = make_tensor_map_2d(&wmap, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(N), row_bytes, row_bytes, 16,
                                  128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&smap, scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, static_cast<uint64_t>(N), G, G * 4, 16,
                                  kGroupsPerBox, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&bmap, biases, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, static_cast<uint64_t>(N), G, G * 4, 16,
                                  kGroupsPerBox, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return bits == 4 ? launch_bits<4>(p, wmap, smap, bmap, x, y, (int)M, (int)N, (int)K, (int)gs, st)
                   : launch_bits<8>(p, wmap, smap, bmap, x, y, (int)M, (int)N, (int)K, (int)gs, st);
}

}  // namespace qmm
