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
#include <type_traits>
#include <utility>

#include "common.cuh"

namespace qmm {
namespace opapi_tc {

constexpr int kMaxWarps = 16;
constexpr int kBox = 2048;           // one TMA box: 16 rows x 128 bytes
constexpr int kStepBytes = 32;       // bytes of a weight row per step of a quad: 4 threads x 8 bytes
constexpr int kStepsPerChunk = 4;    // a box holds 4 steps
constexpr int kGroupsPerBox = 32;    // scales / biases of 32 groups per row in one box
constexpr int kMaxSmem = 227 * 1024;
// boxes per warp's ring.  Deeper rings measured slower where shared memory allowed them (8-bit codes, M <= 2,
// 14336 x 4096: 16.6 and 20.1 us with 8 boxes against 13.9 and 13.1 us with 4): every box requested at the start
// delays the first one.
constexpr int kMaxStages = 4;

namespace dev {
using namespace qmm::dev;

// A loop whose index is a compile-time constant in the body (shared-memory offsets fold into the load
// instructions, the choice of MMA form and of scale component is made at compile time): f(integral_constant<0>) ...
template <typename Fn, int... Is>
__device__ __forceinline__ void static_for_impl(Fn& f, std::integer_sequence<int, Is...>) {
  (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, typename Fn>
__device__ __forceinline__ void static_for(Fn&& f) {
  static_for_impl(f, std::make_integer_sequence<int, N>{});
}

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

// Order of the eight activations of a 16-byte piece in shared memory: the k-slots of one MMA are four codes of one
// packed word per thread of a quad, so a register of the second operand pairs the activations of two codes that
// the first operand takes from one register.
//   kOrderAffine4: (x0,x4) (x2,x6) | (x1,x5) (x3,x7)   one word of 4-bit codes; the second pair meets the codes at bits 4-7
//   kOrderBytes:   (x0,x2) (x1,x3) | (x4,x6) (x5,x7)   two words of 8-bit codes
//   kOrderNatural: (x0,x1) (x2,x3) | (x4,x5) (x6,x7)   codes converted by the hardware, two neighbours per instruction
enum { kOrderAffine4 = 0, kOrderBytes = 1, kOrderNatural = 2 };

// Stages x[M][K] (f16) into shared memory, 8 k (16 bytes) per thread and pass, every global load of a pass issued
// before the first store.  With SUMS, also the sum of each (row, group) into xsum[group * stride + row]: fused into
// the same pass by shuffles when a group is a power-of-two number of lanes (fused_sum), in a fixed order.
// kBatch = loads in flight per thread: with 8, one pass covers 4 rows of K = 4096 with 448 threads.
//
// after_first_loads() runs once, after the first pass's loads have been issued and before anything waits for them:
// the caller requests its TMA boxes there, so that the small activation loads are not queued behind them.
template <int ORDER, bool SUMS, int kBatch, typename Fn>
__device__ __forceinline__ void stage_activations(const __half* __restrict__ x, uint8_t* xs, int row_bytes, int M, int chunks,
                                                  float* xsum, int stride, int lanes_per_group, bool fused_sum,
                                                  Fn after_first_loads) {
  const int tid = threadIdx.x, lane = tid & 31, threads = blockDim.x;
  const int n_it = M * chunks;
  int m = 0, c8 = tid;                                    // i = m * chunks + c8, advanced without a division
  while (c8 >= chunks) { c8 -= chunks; ++m; }
  for (int i0 = tid; i0 - tid < n_it; i0 += threads * kBatch) {   // whole warps stay in the loop for the shuffles
    uint4 v[kBatch];
    int mm[kBatch], cc[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j * threads;
      mm[j] = m;
      cc[j] = c8;
      v[j] = i < n_it ? __ldg(reinterpret_cast<const uint4*>(x) + i) : make_uint4(0, 0, 0, 0);
      c8 += threads;
      while (c8 >= chunks) { c8 -= chunks; ++m; }
    }
    if (i0 == tid) after_first_loads();
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j * threads;
      if (i - lane >= n_it) continue;                     // warp-uniform
      const uint32_t h0 = v[j].x, h1 = v[j].y, h2 = v[j].z, h3 = v[j].w;   // (x0,x1) (x2,x3) (x4,x5) (x6,x7)
      if (i < n_it) {
        uint4 o;
        if (ORDER == kOrderAffine4) {
          o.x = __byte_perm(h0, h2, 0x5410);
          o.y = __byte_perm(h1, h3, 0x5410);
          o.z = __byte_perm(h0, h2, 0x7632);
          o.w = __byte_perm(h1, h3, 0x7632);
        } else if (ORDER == kOrderBytes) {
          o.x = __byte_perm(h0, h1, 0x5410);
          o.y = __byte_perm(h0, h1, 0x7632);
          o.z = __byte_perm(h2, h3, 0x5410);
          o.w = __byte_perm(h2, h3, 0x7632);
        } else {
          o = v[j];
        }
        *reinterpret_cast<uint4*>(xs + mm[j] * row_bytes + cc[j] * 16) = o;
      }
      if (SUMS && fused_sum) {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&h3));
        float p = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        for (int o = 1; o < lanes_per_group; o <<= 1) p += __shfl_xor_sync(0xFFFFFFFFu, p, o);
        if (i < n_it && (cc[j] & (lanes_per_group - 1)) == 0) xsum[(cc[j] / lanes_per_group) * stride + mm[j]] = p;
      }
    }
  }
}

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
         static_cast<size_t>(warps) * 32 * MT * 4 * 4 + static_cast<size_t>(warps) * (kMaxStages + 1) * 8 + 1024;
}

// Picks tiles per CTA, the K split and the ring depth: as many warps as a CTA may have, at most 8 K units per warp
// (one box of scales), at least two boxes of weights per warp (a box is refilled while the next is read).  When the
// staged activations leave too little room, fewer warps.  fixed(warps) = shared memory beside the rings.
template <typename FixedFn>
static bool choose(int64_t tiles_total, int U, int chunks_per_unit, FixedFn fixed, Plan* p) {
  const int ksplit_min = (U + 7) / 8;
  if (ksplit_min > kMaxWarps) return false;
  const int sms = num_sms();
  int tiles = static_cast<int>((tiles_total + sms - 1) / sms);
  if (tiles * ksplit_min > kMaxWarps) tiles = kMaxWarps / ksplit_min;
  int ksplit = kMaxWarps / tiles;
  if (ksplit > U) ksplit = U;
  for (;;) {
    const int warps = tiles * ksplit;
    const size_t fx = fixed(warps);
    const int chunks_per_warp = ((U + ksplit - 1) / ksplit) * chunks_per_unit;
    int stages = fx < static_cast<size_t>(kMaxSmem) ? static_cast<int>((kMaxSmem - fx) / (static_cast<size_t>(warps) * kBox)) : 0;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > chunks_per_warp) stages = chunks_per_warp;
    if (stages >= 2 || (stages == 1 && chunks_per_warp == 1)) {
      p->tiles = tiles;
      p->ksplit = ksplit;
      p->warps = warps;
      p->stages = stages;
      p->grid = static_cast<unsigned>((tiles_total + tiles - 1) / tiles);
      p->smem = fx + static_cast<size_t>(warps) * stages * kBox;
      return true;
    }
    if (ksplit > ksplit_min) ksplit = (ksplit + ksplit_min) / 2;     // first give up the extra K parts, then tiles
    else if (tiles > 1) tiles = (tiles + 1) / 2;
    else return false;
  }
}

// How to cut an affine problem; false when this kernel does not cover it.
static bool plan(int bits, int64_t M, int64_t N, int64_t K, int64_t gs, Plan* p) {
  const int step_k = bits == 4 ? Fmt<4>::kStepK : Fmt<8>::kStepK;
  const int64_t spg = gs / step_k;                       // steps per group
  if (gs % step_k != 0 || (spg != 1 && spg != 2 && spg != 4)) return false;
  if (N % 16 != 0 || K % gs != 0 || K * bits / 8 < 128 || K > (1 << 17)) return false;
  const int64_t G = K / gs;
  if (G % 4 != 0) return false;        // K parts begin on 4 groups: 16 bytes of a scale row, one box of weights
  const int MT = M <= 8 ? 1 : 2;
  return choose(N / 16, static_cast<int>(G / 4), static_cast<int>(spg),
                [&](int warps) { return fixed_smem(bits, warps, static_cast<int>(M), MT, static_cast<int>(K), static_cast<int>(G)); }, p);
}

template <int BITS, int MT, int SPG>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
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
    tma_prefetch_desc(&wmap);
    tma_prefetch_desc(&smap);
    tma_prefetch_desc(&bmap);
    for (int i = 0; i <= stages; ++i) mbar_init(my_bar + i, 1);
    fence_mbar_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  pdl_wait();                 // everything below may read what the previous kernel wrote
  pdl_launch_dependents();
  auto request_boxes = [&]() {
    if (lane == 0 && active) {
      mbar_expect_tx(my_bar + stages, 2 * kBox);
      tma_load_2d(my_sbox, &smap, my_bar + stages, g_begin, n0);
      tma_load_2d(my_sbox + kBox, &bmap, my_bar + stages, g_begin, n0);
      for (int c = 0; c < stages && c < nchunks; ++c) {
        mbar_expect_tx(my_bar + c, kBox);
        tma_load_2d(my_ring + c * kBox, &wmap, my_bar + c, seg_begin + c * 128, n0);
      }
    }
  };

  // ---- activations in MMA slot order, sums per (row, group)
  const int chunks = K / 8;
  const int lanes_per_group = gs / 8;
  const bool fused_sum = lanes_per_group <= 32 && (lanes_per_group & (lanes_per_group - 1)) == 0;
  stage_activations<BITS == 4 ? kOrderAffine4 : kOrderBytes, true, 8>(x, xs, row_bytes, M, chunks, xsum, MT * 8, lanes_per_group,
                                                                  fused_sum, request_boxes);
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
      static_for<kStepsPerChunk>([&](auto s4c) {
        constexpr int s4 = decltype(s4c)::value;
        const uint32_t wa = wbase ^ (s4 << 5);
        const uint2 a = lds64<0>(wa), b = lds64<1024>(wa);
        constexpr bool first = s4 % SPG == 0;
        if constexpr (BITS == 4) {
          static_for<2>([&](auto wic) {
            constexpr int wi = decltype(wic)::value;
            const uint32_t lo = wi ? a.y : a.x, hi = wi ? b.y : b.x;
            const uint32_t lo8 = lo >> 8, hi8 = hi >> 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xq = lds128<s4 * 128 + wi * 16>(xa[mt]);
              if constexpr (wi == 0 && first) {
                mma16816_first(d1[mt], lo & kLo4, hi & kLo4, lo8 & kLo4, hi8 & kLo4, xq.x, xq.y);
                mma16816_first(d16[mt], lo & kHi4, hi & kHi4, lo8 & kHi4, hi8 & kHi4, xq.z, xq.w);
              } else {
                mma16816(d1[mt], lo & kLo4, hi & kLo4, lo8 & kLo4, hi8 & kLo4, xq.x, xq.y);
                mma16816(d16[mt], lo & kHi4, hi & kHi4, lo8 & kHi4, hi8 & kHi4, xq.z, xq.w);
              }
            }
          });
        } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xq = lds128<s4 * 64>(xa[mt]);
            if constexpr (first) mma16816_first(d1[mt], a.x & kByte, b.x & kByte, (a.x >> 8) & kByte, (b.x >> 8) & kByte, xq.x, xq.y);
            else mma16816(d1[mt], a.x & kByte, b.x & kByte, (a.x >> 8) & kByte, (b.x >> 8) & kByte, xq.x, xq.y);
            mma16816(d1[mt], a.y & kByte, b.y & kByte, (a.y >> 8) & kByte, (b.y >> 8) & kByte, xq.z, xq.w);
          }
        }
        if constexpr (s4 % SPG == SPG - 1) {      // a group ends
          // component of the 4-group chunk of scales: static when a chunk of steps holds 4 groups
          const int j = (GPC == 4) ? s4 : ((gq & 3) + s4 / SPG);
          const float sl = sel4(s_lo, j & 3), sh = sel4(s_hi, j & 3), bl = sel4(b_lo, j & 3), bh = sel4(b_hi, j & 3);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float2 xv = lds64f<(s4 / SPG) * MT * 32>(xsa + mt * 32);
            float t0 = d1[mt][0], t1 = d1[mt][1], t2 = d1[mt][2], t3 = d1[mt][3];
            if constexpr (BITS == 4) {
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
      });
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


// ---------------------------------------------------------------------------
// The MX formats (mxfp4, mxfp8: e8m0 scale per 32 k; nvfp4: e4m3 scale per 16 k) on the same skeleton.
// The codes are converted by cvt.rn.f16x2.e2m1x2 / .e4m3x2: one instruction per two neighbouring codes, true
// values (all exact in f16), NaN codes become NaN and reach exactly the output columns of their weight rows
// through the MMA; e8m0 scales by cvt.rn.bf16x2.ue8m0x2 (code 0 = 2^-127, code 255 = NaN).  The activations are therefore staged in their natural order.  mxfp4 and mxfp8 keep one
// accumulator per scale group and apply the decoded e8m0 scale in f32.  nvfp4, whose groups are shorter than
// one MMA's k range per thread, multiplies the converted weights by their scale in f16 before the MMA: the
// product of a 2-bit and a 4-bit significand between 2^-10 and 2688 is exact.
// ---------------------------------------------------------------------------
enum { kMxfp4 = 0, kMxfp8 = 1, kNvfp4 = 2 };

template <int MODE>
struct MxFmt {
  static constexpr int kBits = MODE == kMxfp8 ? 8 : 4;
  static constexpr int kGroup = MODE == kNvfp4 ? 16 : 32;
  static constexpr int kStepK = kStepBytes * 8 / kBits;             // 64 or 32
  static constexpr int kScalesPerStep = kStepK / kGroup;            // mxfp4 2, mxfp8 1, nvfp4 4
  static constexpr int kScalesPerChunk = kStepsPerChunk * kScalesPerStep;
  static constexpr int kUnitSteps = 16 / kScalesPerStep;            // a K part begins on 16 scale bytes
  static constexpr int kXStep = kStepK * 2;
  // mxfp4 takes words t4 and t4 + 4 of a step (one scale group per MMA pair), so a quad reads 64 contiguous
  // bytes of activations, as it does for 8-bit codes; nvfp4 takes words 2 t4 and 2 t4 + 1
  static constexpr int kRowPad = MODE == kNvfp4 ? 16 : 64;
  static constexpr int kOrder = kOrderNatural;
};

namespace dev {
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
  return v;
}
// eight e2m1 codes of a word -> four registers of two f16 each: register j holds codes (2j, 2j + 1), true values
__device__ __forceinline__ void e2m1_to_f16x2(uint32_t w, uint32_t (&r)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(w));
}
// four e4m3 bytes of a word -> bytes (0, 1) and bytes (2, 3) as two f16 each, true values, NaN codes -> NaN
__device__ __forceinline__ void e4m3_to_f16x2(uint32_t w, uint32_t& p01, uint32_t& p23) {
  asm("{\n\t.reg .b16 h0, h1;\n\tmov.b32 {h0, h1}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, h0;\n\tcvt.rn.f16x2.e4m3x2 %1, h1;\n\t}"
      : "=r"(p01), "=r"(p23)
      : "r"(w));
}
// four e8m0 scale codes of a word -> bytes (0, 1) and bytes (2, 3) as two bf16 each: 2^(code - 127), exact
// (code 0 is the bf16 subnormal 2^-127, code 255 is NaN); a bf16 is the upper half of the f32 of the same value
__device__ __forceinline__ void e8m0_to_bf16x2(uint32_t w, uint32_t& p01, uint32_t& p23) {
  asm("{\n\t.reg .b16 h0, h1;\n\tmov.b32 {h0, h1}, %2;\n\t"
      "cvt.rn.bf16x2.ue8m0x2 %0, h0;\n\tcvt.rn.bf16x2.ue8m0x2 %1, h1;\n\t}"
      : "=r"(p01), "=r"(p23)
      : "r"(w));
}
template <int HALF>
__device__ __forceinline__ float bf16_half_as_f32(uint32_t p) {
  return __uint_as_float(HALF ? (p & 0xFFFF0000u) : (p << 16));
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
}  // namespace dev

static size_t mx_fixed_smem(int mode, int warps, int M, int MT, int K) {
  const int pad = mode == kNvfp4 ? 16 : 64;
  return static_cast<size_t>(warps) * kBox + static_cast<size_t>(M) * (2 * K + pad) + static_cast<size_t>(warps) * 32 * MT * 4 * 4 +
         static_cast<size_t>(warps) * (kMaxStages + 1) * 8 + 1024;
}

static bool mx_plan(int mode, int64_t M, int64_t N, int64_t K, Plan* p) {
  const int group = mode == kNvfp4 ? 16 : 32, bits = mode == kMxfp8 ? 8 : 4;
  if (N % 16 != 0 || K % (16 * group) != 0 || K * bits / 8 < 128 || K > (1 << 17)) return false;
  const int MT = M <= 8 ? 1 : 2;
  const int unit_chunks = (mode == kMxfp4 ? 8 : mode == kMxfp8 ? 16 : 4) / kStepsPerChunk;
  return choose(N / 16, static_cast<int>(K / (16 * group)), unit_chunks,      // units of 16 scale bytes
                [&](int warps) { return mx_fixed_smem(mode, warps, static_cast<int>(M), MT, static_cast<int>(K)); }, p);
}

template <int MODE, int MT>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
mx_ring_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
               const __half* __restrict__ x, __half* __restrict__ y, int M, int N, int K, int stages, int tiles, int ksplit,
               int* status) {
  using namespace dev;
  using F = MxFmt<MODE>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int threads = blockDim.x, warps = threads >> 5;
  const int row_bytes = K * 2 + F::kRowPad;
  uint8_t* ring = smem;
  uint8_t* sbox = ring + warps * stages * kBox;
  uint8_t* xs = sbox + warps * kBox;
  float* hand = reinterpret_cast<float*>(xs + M * row_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(hand + warps * 32 * MT * 4);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = warp % tiles, ks = warp / tiles;
  const int n0 = (blockIdx.x * tiles + tile) * 16;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int rho = ((g8 & 3) << 1) | (g8 >> 2);
  const bool active = n0 < N;
  const int U = K / (16 * F::kGroup);
  const int u_begin = (U * ks) / ksplit, u_end = (U * (ks + 1)) / ksplit;
  const int total = active ? (u_end - u_begin) * F::kUnitSteps : 0;
  const int nchunks = total / kStepsPerChunk;
  const int seg_begin = u_begin * (16 * F::kGroup * F::kBits / 8);
  uint8_t* my_ring = ring + warp * stages * kBox;
  uint8_t* my_sbox = sbox + warp * kBox;
  uint64_t* my_bar = bars + warp * (stages + 1);

  if (lane == 0) {
    tma_prefetch_desc(&wmap);
    tma_prefetch_desc(&smap);
    for (int i = 0; i <= stages; ++i) mbar_init(my_bar + i, 1);
    fence_mbar_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  pdl_wait();
  pdl_launch_dependents();
  // mxfp8 measured 4 us slower with 8 loads in flight per thread than with 4 (the other kernels 0.3-0.6 us faster)
  stage_activations<F::kOrder, false, MODE == kMxfp8 ? 4 : 8>(x, xs, row_bytes, M, K / 8, nullptr, 0, 1, false, [&]() {
    if (lane == 0 && active) {
      mbar_expect_tx(my_bar + stages, kBox);
      tma_load_2d(my_sbox, &smap, my_bar + stages, u_begin * 16, n0);
      for (int c = 0; c < stages && c < nchunks; ++c) {
        mbar_expect_tx(my_bar + c, kBox);
        tma_load_2d(my_ring + c * kBox, &wmap, my_bar + c, seg_begin + c * 128, n0);
      }
    }
  });
  __syncthreads();

  float ys[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) ys[mt][i] = 0.f;
  bool ok = true;
  int consumed = 0, requested = stages < nchunks ? stages : nchunks;
  if (active) {
    // this thread's bytes of step 0 within a box (row rho; the 16-byte chunks of a row are XOR-swizzled by rho):
    // 8 bytes at 8 t4 (nvfp4, mxfp8: words 2 t4, 2 t4 + 1) or 4 bytes at 4 t4 and 16 further (mxfp4: words t4, t4 + 4)
    const uint32_t wthread = MODE == kMxfp4 ? rho * 128 + (rho << 4) + (t4 << 2)
                                            : rho * 128 + (((t4 >> 1) ^ rho) << 4) + ((t4 & 1) << 3);
    uint32_t xa[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int row = min(mt * 8 + g8, M - 1);
      xa[mt] = smem_u32(xs) + row * row_bytes + (u_begin * (16 * F::kGroup / 8) + (MODE == kNvfp4 ? 2 * t4 : t4)) * 16;
    }
    const uint32_t sa = smem_u32(my_sbox) + rho * 128;
    ok = wait_box(my_bar + stages, 0, status, 72);
    float d[MT][4];
    if (MODE == kNvfp4) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) d[mt][i] = 0.f;
    }
    const uint32_t sel_t4 = 0x4400u | (t4 << 4) | t4;   // scale byte t4 of a word, twice, into the low half
    int st = 0, prev_st = 0;
    uint32_t phase = 0;
    const uint32_t ring32 = smem_u32(my_ring);
    for (int c = 0; c < nchunks && ok; ++c) {
      ok = wait_box(my_bar + st, phase, status, 73);
      if (!ok) break;
      if (c >= 1 && requested < nchunks) {
        if (lane == 0) {
          mbar_expect_tx(my_bar + prev_st, kBox);
          tma_load_2d(my_ring + prev_st * kBox, &wmap, my_bar + prev_st, seg_begin + requested * 128, n0);
        }
        ++requested;
      }
      // ---- this chunk's scale bytes of rows rho and rho + 8
      // mxfp4, mxfp8: the chunk's e8m0 scales as bf16 pairs (register j = scales 2j, 2j + 1 of the chunk);
      // nvfp4: the words of e4m3 scale bytes
      uint32_t sl[4], sh[4];
      if (MODE == kMxfp4) {
        const uint32_t sq = sa + ((((c >> 1) ^ rho) & 7) << 4) + ((c & 1) << 3);
        const uint2 a = lds64<0>(sq), b = lds64<1024>(sq);
        e8m0_to_bf16x2(a.x, sl[0], sl[1]);
        e8m0_to_bf16x2(a.y, sl[2], sl[3]);
        e8m0_to_bf16x2(b.x, sh[0], sh[1]);
        e8m0_to_bf16x2(b.y, sh[2], sh[3]);
      } else if (MODE == kMxfp8) {
        const uint32_t sq = sa + ((((c >> 2) ^ rho) & 7) << 4) + ((c & 3) << 2);
        e8m0_to_bf16x2(lds32<0>(sq), sl[0], sl[1]);
        e8m0_to_bf16x2(lds32<1024>(sq), sh[0], sh[1]);
      } else {
        const uint32_t sq = sa + (((c ^ rho) & 7) << 4);
        const uint4 a = lds128<0>(sq), b = lds128<1024>(sq);
        sl[0] = a.x; sl[1] = a.y; sl[2] = a.z; sl[3] = a.w;
        sh[0] = b.x; sh[1] = b.y; sh[2] = b.z; sh[3] = b.w;
      }
      const uint32_t wbase = (ring32 + st * kBox) | wthread;
      static_for<kStepsPerChunk>([&](auto s4c) {
        constexpr int s4 = decltype(s4c)::value;
        if constexpr (MODE == kMxfp4) {
          static_for<2>([&](auto wic) {
            constexpr int wi = decltype(wic)::value;
            const uint32_t wa = wbase ^ ((2 * s4 + wi) << 4);
            uint32_t lo[4], hi[4];
            e2m1_to_f16x2(lds32<0>(wa), lo);
            e2m1_to_f16x2(lds32<1024>(wa), hi);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xq = lds128<s4 * 128 + wi * 64>(xa[mt]);
              mma16816_first(d[mt], lo[0], hi[0], lo[1], hi[1], xq.x, xq.y);
              mma16816(d[mt], lo[2], hi[2], lo[3], hi[3], xq.z, xq.w);
            }
            // scale 2 s4 + wi of the chunk: register s4, half wi
            const float fl = bf16_half_as_f32<wi>(sl[s4]), fh = bf16_half_as_f32<wi>(sh[s4]);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              ys[mt][0] = fmaf(fl, d[mt][0], ys[mt][0]);
              ys[mt][1] = fmaf(fl, d[mt][1], ys[mt][1]);
              ys[mt][2] = fmaf(fh, d[mt][2], ys[mt][2]);
              ys[mt][3] = fmaf(fh, d[mt][3], ys[mt][3]);
            }
          });
        } else if constexpr (MODE == kMxfp8) {
          const uint32_t wa = wbase ^ (s4 << 5);
          const uint2 a = lds64<0>(wa), b = lds64<1024>(wa);
          // two registers per word and row: bytes (0, 1) and bytes (2, 3)
          uint32_t ae0, ao0, ae1, ao1, be0, bo0, be1, bo1;
          e4m3_to_f16x2(a.x, ae0, ao0);
          e4m3_to_f16x2(a.y, ae1, ao1);
          e4m3_to_f16x2(b.x, be0, bo0);
          e4m3_to_f16x2(b.y, be1, bo1);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xq = lds128<s4 * 64>(xa[mt]);
            mma16816_first(d[mt], ae0, be0, ao0, bo0, xq.x, xq.y);
            mma16816(d[mt], ae1, be1, ao1, bo1, xq.z, xq.w);
          }
          const float fl = bf16_half_as_f32<(s4 & 1)>(sl[s4 >> 1]), fh = bf16_half_as_f32<(s4 & 1)>(sh[s4 >> 1]);   // scale s4 of the chunk
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            ys[mt][0] = fmaf(fl, d[mt][0], ys[mt][0]);
            ys[mt][1] = fmaf(fl, d[mt][1], ys[mt][1]);
            ys[mt][2] = fmaf(fh, d[mt][2], ys[mt][2]);
            ys[mt][3] = fmaf(fh, d[mt][3], ys[mt][3]);
          }
        } else {
          // nvfp4: this thread's two words of the step lie in the step's 16-k group t4
          const uint32_t wa = wbase ^ (s4 << 5);
          const uint2 a = lds64<0>(wa), b = lds64<1024>(wa);
          // scale byte t4 of the word twice in the low half, converted to (s, s); a NaN code converts to NaN
          uint32_t fl, fh, unused;
          e4m3_to_f16x2(__byte_perm(sl[s4], 0u, sel_t4), fl, unused);
          e4m3_to_f16x2(__byte_perm(sh[s4], 0u, sel_t4), fh, unused);
          static_for<2>([&](auto wic) {
            constexpr int wi = decltype(wic)::value;
            uint32_t lo[4], hi[4];
            e2m1_to_f16x2(wi ? a.y : a.x, lo);
            e2m1_to_f16x2(wi ? b.y : b.x, hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              lo[j] = hmul2_u32(lo[j], fl);
              hi[j] = hmul2_u32(hi[j], fh);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xq = lds128<s4 * 128 + wi * 16>(xa[mt]);
              mma16816(d[mt], lo[0], hi[0], lo[1], hi[1], xq.x, xq.y);
              mma16816(d[mt], lo[2], hi[2], lo[3], hi[3], xq.z, xq.w);
            }
          });
        }
      });
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xa[mt] += kStepsPerChunk * F::kXStep;
      __syncwarp();
      ++consumed;
      prev_st = st;
      if (++st == stages) { st = 0; phase ^= 1; }
    }
    if (!ok) {
      for (int c = consumed + 1; c < requested; ++c) {
        if (++st == stages) { st = 0; phase ^= 1; }
        mbar_wait_relaxed_warp(my_bar + st, phase, nullptr, 0);
      }
    }
    if (MODE == kNvfp4) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) ys[mt][i] = d[mt][i];
    }
  }
  float* slot = hand + (warp * 32 + lane) * MT * 4;
  if (ks != 0 && active) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) slot[mt * 4 + i] = ys[mt][i];
  }
  __syncthreads();
  if (ks == 0 && active) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = ys[mt][i];
        for (int o = 1; o < ksplit; ++o) v += hand[((o * tiles + tile) * 32 + lane) * MT * 4 + mt * 4 + i];
        const int n = n0 + rho + ((i >> 1) << 3), m = mt * 8 + 2 * t4 + (i & 1);
        if (m < M) y[static_cast<size_t>(m) * N + n] = __float2half_rn(v);
      }
    }
  }
}

template <int MODE, int MT>
static int mx_launch_one(const Plan& p, const CUtensorMap& wmap, const CUtensorMap& smap, const void* x, void* y, int M, int N,
                         int K, cudaStream_t stream) {
  static std::atomic<uint64_t> configured{0};
  auto kernel = mx_ring_kernel<MODE, MT>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxSmem, configured)) return rc;
  cudaError_t e = launch_pdl(kernel, dim3(p.grid), dim3(p.warps * 32), p.smem, stream, wmap, smap, static_cast<const __half*>(x),
                             static_cast<__half*>(y), M, N, K, p.stages, p.tiles, p.ksplit, device_status_word());
  if (e != cudaSuccess) return set_error(QMM_ERR_CUDA, "mx_qgemm_f16 (TMA ring): launch failed: %s", cudaGetErrorString(e));
  return QMM_OK;
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

// The same for the MX modes (0 mxfp4, 1 mxfp8, 2 nvfp4): f16 activations, 1 <= M <= 16, K a multiple of 16 scale
// groups, 16-byte aligned operands.
bool mx_ring_covers(int64_t M, int64_t N, int64_t K, int mode, int dtype, const void* x, const void* w, const void* scales) {
  using namespace opapi_tc;
  if (mode < 0 || mode > 2 || dtype != QMM_F16 || M < 1 || M > 16) return false;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(scales, 16)) return false;
  Plan p;
  return mx_plan(mode, M, N, K, &p);
}

int mx_ring_launch(int mode, const void* x, const void* w, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                   void* stream) {
  using namespace opapi_tc;
  Plan p;
  QMM_REQUIRE(mx_plan(mode, M, N, K, &p), QMM_ERR_UNSUPPORTED, "mx_ring_launch: shape not covered");
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "qmm_mx_matmul: an earlier kernel gave up a wait (status 0x%x); "
                     "call qmm_clear_device_status() after handling it", st);
  CUtensorMap wmap, smap;
  const int bits = mode == kMxfp8 ? 8 : 4, group = mode == kNvfp4 ? 16 : 32;
  const uint64_t row_bytes = static_cast<uint64_t>(K) * bits / 8, srow = static_cast<uint64_t>(K / group);
  if (int rc = make_tensor_map_2d(&wmap, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(N), row_bytes, row_bytes, 16,
                                  128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&smap, scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(N), srow, srow, 16, 128,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
  if (mode == kMxfp4)
    return M <= 8 ? mx_launch_one<kMxfp4, 1>(p, wmap, smap, x, y, m, n, k, st) : mx_launch_one<kMxfp4, 2>(p, wmap, smap, x, y, m, n, k, st);
  if (mode == kMxfp8)
    return M <= 8 ? mx_launch_one<kMxfp8, 1>(p, wmap, smap, x, y, m, n, k, st) : mx_launch_one<kMxfp8, 2>(p, wmap, smap, x, y, m, n, k, st);
  return M <= 8 ? mx_launch_one<kNvfp4, 1>(p, wmap, smap, x, y, m, n, k, st) : mx_launch_one<kNvfp4, 2>(p, wmap, smap, x, y, m, n, k, st);
}

}  // namespace qmm
