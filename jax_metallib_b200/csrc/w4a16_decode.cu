// int4 group-wise (g128, asymmetric) weight-only matmul at decode sizes (M <= 32).
//
//   y[M,N] = bf16( x[M,K] @ ((q[K,N] - z[K/128,N]) * s[K/128,N]) )
//
// HBM-bound: the packed weights (K*N/2 bytes) are read exactly once.  The work
// is cut into units of one 256-column block x one 128-k group (two 64-row x
// 128-byte TMA boxes side by side, 16 KB: 256 contiguous bytes per DRAM row
// stream measurably faster than 128); consecutive units are dealt evenly to a
// grid of resident CTAs (two per SM).
//
// Per CTA: a producer warp issues the loads of a unit (packed weights with the
// 128-byte swizzle, bulk copies of scales and zero points, a TMA box of the
// group's activations) into an mbarrier ring, and two units later turns those
// activations into the MMA's operand: f16, scaled per (row, group) by a power
// of two so that any bf16 magnitude fits, odd k divided by 16, every four k
// permuted to fragment order, written back in place.
// Eight consumer warps each own 32 columns.  A consumer reads the tile with
// ldmatrix.trans, which turns the k-pair-per-byte layout into registers that
// hold (same column, two k) in their 16-bit halves; one AND per register
// leaves the f16 subnormal q * 2^-24 (low nibbles) or 16 q * 2^-24 (high
// nibbles, no shift needed: the factor 16 is what the activations of odd k
// were divided by), and mma.sync.m16n8k16 (f16, f32 accumulate) takes the
// weights as its 16-row operand and the activations as its 8-column operand:
// one MMA per 256 weights for M <= 8.  The sum of a row's scaled activations
// over each 64-k half of the group, the factor of the zero point, is computed
// once by the producer while it converts them.  Five integer instructions per
// eight weights and nothing else.  Per group:
//   y += s[g,n] * 2^e[m,g] * (2^24 * acc - z[g,n] * sum_k x).
// Partial sums of CTAs sharing a column block meet in the caller's workspace;
// the last CTA to arrive adds them in a fixed order (deterministic result) and
// writes bf16.  The workspace counters are left at zero.
//
// Launch overlap: the kernel is launched with programmatic stream
// serialization, so its CTAs may start while the previous kernel on the stream
// drains.  Everything that can depend on earlier work (activations, output,
// workspace) is touched only after griddepcontrol.wait; when the caller states
// that the weights are static, their first loads are issued before that wait.
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <utility>

#include "common.cuh"

namespace qmm {

int w4a16_tcgen05(const uint16_t* x, const uint8_t* wq, const uint16_t* scales, const uint8_t* zeros,
                  int zeros_packed, uint16_t* y, int64_t M, int64_t N, int64_t K, uint32_t flags,
                  cudaStream_t stream);

namespace w4 {

constexpr int kDecodeMaxM = 32;      // rows the decode kernel covers; larger M goes to the tcgen05 GEMM
constexpr int kColsPerBlock = 256;   // columns per unit: two 128-byte TMA boxes
constexpr int kGroup = 128;          // k per unit
constexpr int kRowsPerUnit = 64;     // packed byte-rows per unit
constexpr int kRowsPerHalf = 32;     // a CTA's first and last unit may be half units (TMA boxes are 32 rows)
constexpr int kConsumerWarps = 8;    // 32 columns (two 16-byte chunks) each
constexpr int kThreads = (kConsumerWarps + 2) * 32;  // consumers, the load-issuing warp, the activation-converting warp
constexpr int kXRowBytes = 256;      // 128 16-bit activations; 16-byte chunks XOR-swizzled by (row & 3) << 1
constexpr int kBoxBytes = kRowsPerUnit * 128;  // 8192: one 128-column half of a unit
constexpr int kHalfBoxBytes = kRowsPerHalf * 128;

template <int MT>
struct Smem {
  static constexpr int kW = 2 * kBoxBytes;                 // 16384
  static constexpr int kS = kColsPerBlock * 2;             // 512
  static constexpr int kZ = kColsPerBlock;                 // 256 (128 used when packed)
  static constexpr int kF = 128;                           // per-row power-of-two factors (MT*8 floats)
  static constexpr int kXS = 256;                          // per-row sums of the scaled activations, one per 64-k half (MT*8 x 2 floats)
  static constexpr int kX = MT * 8 * kXRowBytes;           // also the byte count of the TMA box
  static constexpr int kOffS = kW;
  static constexpr int kOffZ = kOffS + kS;
  static constexpr int kOffF = kOffZ + kZ;
  static constexpr int kOffXS = kOffF + kF;
  static constexpr int kOffX = 17664;                      // multiple of 256 (the swizzle uses address bits 5-7)
  static constexpr int kStage = ((kOffX + kX + 1023) / 1024) * 1024;
  static constexpr int kMinBlocks = (MT <= 2) ? 2 : 1;     // resident CTAs per SM
  static constexpr int kStages = (MT <= 2) ? 5 : 8;
  static constexpr int kBarBytes = 1024;
  static constexpr int kTotal = kStages * kStage + kBarBytes + 1024;  // + alignment slack
  static_assert(kOffXS + kXS <= kOffX, "stage layout overlaps");
};

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dev::smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(dev::smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// not volatile: a pure function of its operands, so that the compiler may interleave the MMAs of a slab with the
// conversion of the next one
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}


// f(integral_constant<0>) ... f(integral_constant<N-1>): a loop whose index is a compile-time constant in the body
template <typename Fn, int... Is>
__device__ __forceinline__ void static_for_impl(Fn& f, std::integer_sequence<int, Is...>) {
  (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, typename Fn>
__device__ __forceinline__ void static_for(Fn&& f) {
  static_for_impl(f, std::make_integer_sequence<int, N>{});
}

// CTA that owns unit u when U units are dealt to P CTAs as [i*U/P, (i+1)*U/P).
__device__ __forceinline__ int cta_of_unit(long long u, int P, int U) {
  return static_cast<int>(((u + 1) * P - 1) / U);
}

// Eight packed weights of one register -> four f16x2 MMA operand registers
// (columns c and c+1, k pairs (4t, 4t+2) and (4t+1, 4t+3) of the slab).  A
// nibble left in place is the f16 subnormal q * 2^-24 (low nibble) or
// 16 q * 2^-24 (high nibble; the factor 16 is what the activations of odd k
// were divided by): no offset to remove, exact products.
__device__ __forceinline__ void dequant8(uint32_t w, uint32_t (&r)[4]) {
  const uint32_t t = w >> 8;
  r[0] = w & 0x000F000Fu;  // bytes 0/2, low nibbles
  r[1] = w & 0x00F000F0u;  // bytes 0/2, high nibbles (x16)
  r[2] = t & 0x000F000Fu;  // bytes 1/3
  r[3] = t & 0x00F000F0u;
}

template <int MT, bool ZP_PACKED>
__global__ void __launch_bounds__(kThreads, Smem<MT>::kMinBlocks)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                    const uint16_t* __restrict__ scales, const uint8_t* __restrict__ zeros,
                    uint16_t* __restrict__ y, float* __restrict__ ws_partial,
                    int* __restrict__ ws_counter, int M, int N, int K, int G, int U, int max_slots,
                    int static_weights, int* status
                    ) {
  using L = Smem<MT>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * L::kStage);
  uint64_t* empty = full + S;
  uint64_t* xraw = empty + S;      // raw activations of the group have landed

  grid_launch_dependents();  // the next kernel on the stream may start its own prologue

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int P = gridDim.x;
  // The range of this CTA in half units (64 k); whole units in between.
  const int h_begin = static_cast<int>((static_cast<long long>(blockIdx.x) * 2 * U) / P);
  const int h_end = static_cast<int>((static_cast<long long>(blockIdx.x + 1) * 2 * U) / P);
  const int u_begin = h_begin >> 1;
  const int u_end = (h_end + 1) >> 1;
  const int n_units = u_end - u_begin;
  // halves of unit number `it` of this CTA that belong to it: [first, last)
  auto half_lo = [&](int it) { return (it == 0) ? (h_begin & 1) : 0; };
  auto half_hi = [&](int it) { return (it == n_units - 1 && (h_end & 1)) ? 1 : 2; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      dev::mbar_init(&full[s], 2);                // TMA transaction arrive + activation staging
      dev::mbar_init(&empty[s], kConsumerWarps);  // one arrive per consumer warp
      dev::mbar_init(&xraw[s], 1);
    }
    dev::fence_mbar_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      dev::tma_prefetch_desc(&wmap);
      dev::tma_prefetch_desc(&xmap);
    }
    const uint64_t policy = dev::policy_evict_first();
    // weights, scales and zero points of a unit (one elected lane)
    auto issue_weights = [&](int s, int c, int g, int it) {
      uint8_t* st = smem + s * L::kStage;
      const int col0 = c * kColsPerBlock;
      const int cols = min(kColsPerBlock, N - col0);  // 128 in a trailing half block
      const uint32_t sbytes = cols * 2;
      const uint32_t zbytes = ZP_PACKED ? cols / 2 : cols;
      const int hl = half_lo(it), hh = half_hi(it);
      dev::mbar_expect_tx(&full[s], (hh - hl) * 2 * kHalfBoxBytes + sbytes + zbytes);
      for (int h = hl; h < hh; ++h) {
        const int row = g * kRowsPerUnit + h * kRowsPerHalf;
        dev::tma_load_2d_hint(st + h * kHalfBoxBytes, &wmap, &full[s], col0, row, policy);
        dev::tma_load_2d_hint(st + kBoxBytes + h * kHalfBoxBytes, &wmap, &full[s], col0 + 128, row, policy);
      }
      bulk_copy_g2s(st + L::kOffS, scales + static_cast<size_t>(g) * N + col0, sbytes, &full[s]);
      const uint8_t* zsrc = ZP_PACKED ? zeros + static_cast<size_t>(g) * (N / 2) + col0 / 2
                                      : zeros + static_cast<size_t>(g) * N + col0;
      bulk_copy_g2s(st + L::kOffZ, zsrc, zbytes, &full[s]);
    };
    auto issue_x = [&](int s, int g) {
      uint8_t* st = smem + s * L::kStage;
      dev::mbar_expect_tx(&xraw[s], L::kX);  // rows beyond M are zero-filled by the TMA unit
      dev::tma_load_2d(st + L::kOffX, &xmap, &xraw[s], g * kGroup, 0);
    };
    int c = (n_units > 0) ? u_begin / G : 0;
    int g = (n_units > 0) ? u_begin - c * G : 0;
    // Static weights do not depend on earlier kernels: fill the ring with them
    // before waiting for those kernels to finish.
    int prefetched = 0;
    if (static_weights) {
      prefetched = n_units < S ? n_units : S;
      if (lane == 0) {
        int cc = c, gg = g;
        for (int i = 0; i < prefetched; ++i) {
          issue_weights(i, cc, gg, i);
          if (++gg == G) { gg = 0; ++cc; }
        }
      }
    }
    grid_dependency_wait();
    int s_issue = 0;
    uint32_t ph_issue = 0;
    for (int it = 0; it < n_units; ++it) {
      if (it >= prefetched) {
        if (!dev::mbar_wait_relaxed_warp(&empty[s_issue], ph_issue ^ 1, status, 1)) break;
        if (lane == 0) issue_weights(s_issue, c, g, it);
      }
      if (lane == 0) issue_x(s_issue, g);
      if (++g == G) { g = 0; ++c; }
      if (++s_issue == S) { s_issue = 0; ph_issue ^= 1; }
    }
  } else if (warp == kConsumerWarps + 1) {
    // ------------------------- activation converter -----------------------
    // A warp of its own: the conversion of a unit's activations is on the path of every unit
    // (the consumers need it), so it must not queue behind the issue of the next unit's loads.
    constexpr int kPasses = MT * 4;  // a pass = 2 rows x 16 lanes x 16 bytes
    grid_dependency_wait();
    int s_conv = 0;
    uint32_t ph_conv = 0;
    for (int it = 0; it < n_units; ++it) {
      {
        if (!dev::mbar_wait_relaxed_warp(&xraw[s_conv], ph_conv, status, 4)) break;
        uint8_t* st = smem + s_conv * L::kStage;
        float* fac = reinterpret_cast<float*>(st + L::kOffF);
        float* xsum_row = reinterpret_cast<float*>(st + L::kOffXS);
        uint4 v[kPasses];
#pragma unroll
        for (int p = 0; p < kPasses; ++p) {
          const int row = p * 2 + (lane >> 4);
          v[p] = *reinterpret_cast<const uint4*>(st + L::kOffX + row * kXRowBytes + (lane & 15) * 16);
        }
        __syncwarp();  // every raw chunk is in registers before any is overwritten
#pragma unroll
        for (int p = 0; p < kPasses; ++p) {
          const int row = p * 2 + (lane >> 4);
          // largest magnitude of the row's 128 values, from the bf16 bit patterns
          uint32_t mx = __vmaxu2(__vmaxu2(v[p].x & 0x7FFF7FFFu, v[p].y & 0x7FFF7FFFu),
                                 __vmaxu2(v[p].z & 0x7FFF7FFFu, v[p].w & 0x7FFF7FFFu));
          mx = max(mx & 0xFFFFu, mx >> 16);
#pragma unroll
          for (int off = 8; off >= 1; off >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
          // scale the row by 2^(135 - e) so that |x| < 2^9 in f16 whatever its bf16
          // exponent e was; the inverse goes to the consumers.  Degenerate rows
          // (all tiny, or inf/NaN present) are passed through unscaled.
          const uint32_t e8 = mx >> 7;
          const bool scaled = (e8 >= 16u) && (e8 < 255u);
          const float mul = scaled ? __uint_as_float((262u - e8) << 23) : 1.0f;
          const float inv = scaled ? __uint_as_float((e8 - 8u) << 23) : 1.0f;
          const float e0 = __uint_as_float(v[p].x << 16) * mul, o0 = __uint_as_float(v[p].x & 0xFFFF0000u) * mul;
          const float e1 = __uint_as_float(v[p].y << 16) * mul, o1 = __uint_as_float(v[p].y & 0xFFFF0000u) * mul;
          const float e2 = __uint_as_float(v[p].z << 16) * mul, o2 = __uint_as_float(v[p].z & 0xFFFF0000u) * mul;
          const float e3 = __uint_as_float(v[p].w << 16) * mul, o3 = __uint_as_float(v[p].w & 0xFFFF0000u) * mul;
          // sums of the row's scaled activations over each 64-k half of the group (a CTA may own
          // only one half of a unit): what the zero point multiplies, computed once per (row, group)
          // here instead of once per consumer warp on the tensor cores.  Eight lanes hold a half.
          float xs = ((e0 + o0) + (e1 + o1)) + ((e2 + o2) + (e3 + o3));
#pragma unroll
          for (int off = 4; off >= 1; off >>= 1) xs += __shfl_xor_sync(0xFFFFFFFFu, xs, off);
          const uint32_t w0 = pack_f16x2(e0, o0 * 0.0625f);
          const uint32_t w1 = pack_f16x2(e1, o1 * 0.0625f);
          const uint32_t w2 = pack_f16x2(e2, o2 * 0.0625f);
          const uint32_t w3 = pack_f16x2(e3, o3 * 0.0625f);
          // every 4 consecutive k go from (0,1,2,3) to (0,2,1,3): the order the
          // MMA fragments of the consumers read them in
          uint4 o;
          o.x = __byte_perm(w0, w1, 0x5410);
          o.y = __byte_perm(w0, w1, 0x7632);
          o.z = __byte_perm(w2, w3, 0x5410);
          o.w = __byte_perm(w2, w3, 0x7632);
          const int chunk = (lane & 15) ^ ((row & 3) << 1);
          *reinterpret_cast<uint4*>(st + L::kOffX + row * kXRowBytes + chunk * 16) = o;
          if ((lane & 15) == 0) fac[row] = inv;
          if ((lane & 7) == 0) xsum_row[2 * row + ((lane >> 3) & 1)] = xs;
        }
        __syncwarp();
        if (lane == 0) dev::mbar_arrive(&full[s_conv]);
        if (++s_conv == S) { s_conv = 0; ph_conv ^= 1; }
      }
    }
  } else {
    // ------------------------------ consumers -----------------------------
    grid_dependency_wait();    // before anything is written to the output or the workspace
    const int g8 = lane >> 2;  // 0..7
    const int t4 = lane & 3;   // 0..3
    // ldmatrix: lane l addresses row 32h + l of this warp's box, 16-byte chunk ch (swizzled by the row)
    const int ch0 = 2 * (warp & 3);
    const uint32_t ld_base = (warp >> 2) * kBoxBytes + lane * 128;
    const uint32_t ld_off0 = ld_base + ((ch0 ^ (lane & 7)) << 4);
    const uint32_t ld_off1 = ld_base + (((ch0 + 1) ^ (lane & 7)) << 4);
    // activation fragment: row g8 (+8 per tile), chunk 2*slab + t4/2 swizzled by the row,
    // 8-byte half t4 & 1.  Address bits 5-7 carry the chunk, so the slab is XOR-ed in.
    const uint32_t x_off = L::kOffX + g8 * kXRowBytes + ((t4 >> 1) << 4) + ((t4 & 1) << 3) +
                           ((g8 & 3) << 5);
    const int lc = warp * 32 + 2 * g8;  // first column pair of this thread inside the block (second: +16)
    float yacc[2][MT][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) yacc[j][mt][i] = 0.f;

    // Hand this warp's 32 columns of the finished column block over.  CTAs that
    // share the block each write a partial tile; every warp counts arrivals on
    // its own counter, and the warp that arrives last adds the partial tiles of
    // its columns in slot order (so the result does not depend on arrival
    // order) and writes bf16.  No CTA-wide rendezvous is involved.
    auto flush = [&](int c) {
      const int first = cta_of_unit(static_cast<long long>(c) * 2 * G, P, 2 * U);
      const int last = cta_of_unit(static_cast<long long>(c) * 2 * G + 2 * G - 1, P, 2 * U);
      const int nslots = last - first + 1;
      const int col0 = c * kColsPerBlock;
      if (nslots == 1) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const int m = mt * 8 + 2 * t4 + r;
              const int col = col0 + lc + 16 * j;
              if (m < M && col < N)
                *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(m) * N + col) =
                    dev::pack_bf16x2(yacc[j][mt][r], yacc[j][mt][2 + r]);
            }
        return;
      }
      const int slot = static_cast<int>(blockIdx.x) - first;
      float* part = ws_partial + (static_cast<size_t>(c) * max_slots + slot) * (MT * 8) * kColsPerBlock;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int m = mt * 8 + 2 * t4 + r;
            if (m < M)
              __stcg(reinterpret_cast<float2*>(part + m * kColsPerBlock + lc + 16 * j),
                     make_float2(yacc[j][mt][r], yacc[j][mt][2 + r]));
          }
      __syncwarp();
      int is_last = 0;
      if (lane == 0) {
        __threadfence();  // the warp's partial tile is visible before its arrival is
        is_last = (atomicAdd(&ws_counter[c * kConsumerWarps + warp], 1) + 1 == nslots);
        if (is_last) __threadfence();
      }
      is_last = __shfl_sync(0xFFFFFFFFu, is_last, 0);
      if (!is_last) return;
      const float* base = ws_partial + static_cast<size_t>(c) * max_slots * (MT * 8) * kColsPerBlock;
      const int wcol = warp * 32 + lane;  // one column per lane
      // four rows x four slots of loads in flight; slots are always added in
      // ascending order, so the rounding does not depend on who arrived last
      for (int m0 = 0; m0 < M; m0 += 4) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        for (int sl0 = 0; sl0 < nslots; sl0 += 4) {
          float v[4][4];
#pragma unroll
          for (int ds = 0; ds < 4; ++ds)
#pragma unroll
            for (int r = 0; r < 4; ++r)
              v[ds][r] = (sl0 + ds < nslots && m0 + r < M)
                             ? __ldcg(base + (static_cast<size_t>(sl0 + ds) * (MT * 8) + m0 + r) * kColsPerBlock + wcol)
                             : 0.f;
#pragma unroll
          for (int ds = 0; ds < 4; ++ds)
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] += v[ds][r];
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float b = __shfl_down_sync(0xFFFFFFFFu, a[r], 1);
          if (m0 + r < M && !(lane & 1) && col0 + wcol < N)
            *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(m0 + r) * N + col0 + wcol) =
                dev::pack_bf16x2(a[r], b);
        }
      }
      __syncwarp();
      if (lane == 0) ws_counter[c * kConsumerWarps + warp] = 0;
    };

    int c = (n_units > 0) ? u_begin / G : 0;
    int g = (n_units > 0) ? u_begin - c * G : 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int it = 0; it < n_units; ++it) {
      if (!dev::mbar_wait_relaxed_warp(&full[s], ph, status, 2)) {
        ok = false;
        break;
      }
      const uint8_t* st = smem + s * L::kStage;
      const uint32_t st_addr = dev::smem_u32(st);

      // per-group constants of this thread's four columns (pairs lc, lc+16)
      float sc[2][2];
      float zf[2][2];  // zero points
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = lc + 16 * j;
        const uint32_t s2 = *reinterpret_cast<const uint32_t*>(st + L::kOffS + col * 2);
        sc[j][0] = __uint_as_float(s2 << 16);
        sc[j][1] = __uint_as_float(s2 & 0xFFFF0000u);
        uint32_t z0, z1;
        if (ZP_PACKED) {
          const uint32_t zb = st[L::kOffZ + (col >> 1)];
          z0 = zb & 0xFu;
          z1 = zb >> 4;
        } else {
          const uint32_t zb = *reinterpret_cast<const uint16_t*>(st + L::kOffZ + col);
          z0 = zb & 0xFFu;
          z1 = zb >> 8;
        }
        zf[j][0] = __uint_as_float(0x4B000000u | z0) - 8388608.f;
        zf[j][1] = __uint_as_float(0x4B000000u | z1) - 8388608.f;
      }

      float acc[2][MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[0][mt][i] = 0.f;
          acc[1][mt][i] = 0.f;
        }
      const uint32_t xb = st_addr + x_off;

      const int hl = half_lo(it), hh = half_hi(it);
      // both loops run over compile-time indices, so that the slab's XOR into the activation address and the
      // choice of ldmatrix register are constants of each copy of the body
      static_for<2>([&](auto hc) {
        constexpr int h = decltype(hc)::value;
        if (h < hl || h >= hh) return;  // the other half of a boundary unit belongs to a neighbour CTA
        uint32_t wa[4], wb[4];
        ldmatrix_x4_trans(st_addr + ld_off0 + h * 4096, wa);
        ldmatrix_x4_trans(st_addr + ld_off1 + h * 4096, wb);
        static_for<4>([&](auto qc) {
          constexpr int q = decltype(qc)::value;
          constexpr int slab = 4 * h + q;
          uint32_t xf[MT][2];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];"
                         : "=r"(xf[mt][0]), "=r"(xf[mt][1])
                         : "r"((xb ^ (slab << 5)) + mt * 8 * kXRowBytes));
          uint32_t r[4];
          dequant8(wa[q], r);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            mma_f16_16816(acc[0][mt], r[0], r[2], r[1], r[3], xf[mt][0], xf[mt][1]);
          dequant8(wb[q], r);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            mma_f16_16816(acc[1][mt], r[0], r[2], r[1], r[3], xf[mt][0], xf[mt][1]);
        });
      });
      // group epilogue: per pair this thread holds columns (c, c+1) for rows
      // (2t, 2t+1) of each 8-row tile
      const float* fac = reinterpret_cast<const float*>(st + L::kOffF);
      const float* xsr = reinterpret_cast<const float*>(st + L::kOffXS);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float2 f = *reinterpret_cast<const float2*>(fac + mt * 8 + 2 * t4);
        // rows 2t, 2t+1: (first half, second half) each; only the halves this CTA multiplied count
        const float4 xh = *reinterpret_cast<const float4*>(xsr + 2 * (mt * 8 + 2 * t4));
        const float2 xs = make_float2((hl == 0 ? xh.x : 0.f) + (hh == 2 ? xh.y : 0.f),
                                      (hl == 0 ? xh.z : 0.f) + (hh == 2 ? xh.w : 0.f));
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          // sum_k (q - z) x = acc * 2^24 - z * sum_k x (the weights went in as q * 2^-24)
          const float v0 = fmaf(acc[j][mt][0], 16777216.f, -zf[j][0] * xs.x);
          const float v1 = fmaf(acc[j][mt][1], 16777216.f, -zf[j][0] * xs.y);
          const float v2 = fmaf(acc[j][mt][2], 16777216.f, -zf[j][1] * xs.x);
          const float v3 = fmaf(acc[j][mt][3], 16777216.f, -zf[j][1] * xs.y);
          yacc[j][mt][0] = fmaf(sc[j][0] * f.x, v0, yacc[j][mt][0]);
          yacc[j][mt][1] = fmaf(sc[j][0] * f.y, v1, yacc[j][mt][1]);
          yacc[j][mt][2] = fmaf(sc[j][1] * f.x, v2, yacc[j][mt][2]);
          yacc[j][mt][3] = fmaf(sc[j][1] * f.y, v3, yacc[j][mt][3]);
        }
      }
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(&empty[s]);
      if (++s == S) { s = 0; ph ^= 1; }
      if (++g == G) {
        // the column block is complete as far as this CTA is concerned
        g = 0;
        flush(c);
        ++c;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) yacc[j][mt][i] = 0.f;
      }
    }
    if (ok && n_units > 0 && g != 0) flush(c);
  }
}

// One launch path for both entry points: `status` is where a bounded wait that
// gives up is recorded (may be null).
template <int MT, bool ZP>
static int launch(const CUtensorMap& wmap, const CUtensorMap& xmap, const uint16_t* scales,
                  const uint8_t* zeros, uint16_t* y, float* ws_partial, int* ws_counter, int M, int N,
                  int K, int G, int U, int P, int max_slots, int static_weights, int* status,
                  cudaStream_t stream) {
  using L = Smem<MT>;
  static std::atomic<uint64_t> configured{0};  // per device (one mask per template instance)
  auto kern = w4a16_decode_kernel<MT, ZP>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kTotal, configured)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(P);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, wmap, xmap, scales, zeros, y, ws_partial, ws_counter, M,
                                  N, K, G, U, max_slots, static_weights, status));
  return QMM_OK;
}

static int blocks_per_sm(int M) { return M <= 16 ? 2 : 1; }
// Small problems get at least this many units per CTA so that few CTAs share a column block.
// Measured on the decode step (4096x6144, 4096x4096, 4096x28672, 14336x4096 at M = 8):
// 2 and 3 units 3.35 ms per step, 4 units 3.26 ms, 6 units 3.50 ms.
constexpr int kMinUnitsPerCta = 4;
static int grid_size(int U, int M) {
  // every CTA resident at once; small problems get at least four units per CTA
  // so that few CTAs share a column block
  const int p = blocks_per_sm(M) * num_sms();
  const int mu = kMinUnitsPerCta;
  const int q = (U + mu - 1) / mu;
  return q < p ? q : p;
}
static int slots_for(int G, int U, int P) {
  // a column block of G units is shared by at most ceil(G*P/U) + 1 CTAs
  return static_cast<int>((static_cast<long long>(G) * P + U - 1) / U) + 1;
}
// One arrival counter per (column block, consumer warp).  The counters occupy a
// fixed-size header of the workspace so that calls with different shapes can
// share one workspace: only this header has to be zero between calls, and every
// call leaves it zero.
constexpr int kMaxColBlocks = 2048;
static size_t counter_bytes(int /*C*/) { return static_cast<size_t>(kMaxColBlocks) * kConsumerWarps * sizeof(int); }
static int rows_padded(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : 32); }
static int col_blocks(int64_t N) { return static_cast<int>((N + kColsPerBlock - 1) / kColsPerBlock); }

// Shared body of the two entry points: argument checks, tensor maps, launch.
static int run(const char* name, const uint16_t* x, const uint8_t* wq, const uint16_t* scales,
               const uint8_t* zeros, int zeros_packed, uint16_t* y, int64_t M, int64_t N, int64_t K,
               void* workspace, unsigned flags, int* status, cudaStream_t st) {
  const int G = static_cast<int>(K / kGroup);
  const int C = col_blocks(N);
  const int U = G * C;
  const int P = grid_size(U, static_cast<int>(M));
  (void)name;
  const int slots = slots_for(G, U, P);
  const size_t counters = counter_bytes(C);
  int* ws_counter = static_cast<int*>(workspace);
  float* ws_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counters);

  CUtensorMap wmap, xmap;
  if (int rc = make_tensor_map_2d(&wmap, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                                  static_cast<uint64_t>(K / 2), static_cast<uint64_t>(N),
                                  static_cast<uint64_t>(N), kRowsPerHalf, 128,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // activations: [M, K] bf16, one box = (8, 16 or 32 rows) x one 128-k group, rows past M read as zero
  if (int rc = make_tensor_map_2d(&xmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                  static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                                  static_cast<uint64_t>(K) * 2, rows_padded(static_cast<int>(M)),
                                  kGroup, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
  const int sw = (flags & QMM_W4_STATIC_WEIGHTS) ? 1 : 0;
#define QMM_W4_LAUNCH(MT)                                                                         \
  (zeros_packed ? launch<MT, true>(wmap, xmap, scales, zeros, y, ws_partial, ws_counter, m, n, k, \
                                   G, U, P, slots, sw, status, st)                                \
                : launch<MT, false>(wmap, xmap, scales, zeros, y, ws_partial, ws_counter, m, n,   \
                                    k, G, U, P, slots, sw, status, st))
  if (M <= 8) return QMM_W4_LAUNCH(1);
  if (M <= 16) return QMM_W4_LAUNCH(2);
  return QMM_W4_LAUNCH(4);
#undef QMM_W4_LAUNCH
}

static int check_args(const char* name, const void* x, const void* wq, const void* scales,
                      const void* zeros, const void* y, int64_t M, int64_t N, int64_t K,
                      int64_t group, int64_t max_m) {
  QMM_REQUIRE(x && wq && scales && zeros && y, QMM_ERR_INVALID_ARGUMENT, "%s: null tensor pointer", name);
  QMM_REQUIRE(group == kGroup, QMM_ERR_UNSUPPORTED, "%s: group must be 128, got %lld", name,
              (long long)group);
  QMM_REQUIRE(M >= 1 && M <= max_m, QMM_ERR_UNSUPPORTED, "%s: covers 1 <= M <= %lld, got %lld", name,
              (long long)max_m, (long long)M);
  QMM_REQUIRE(N >= 128 && N % 128 == 0 && K >= kGroup && K % kGroup == 0, QMM_ERR_UNSUPPORTED,
              "%s: N (%lld) and K (%lld) must be positive multiples of 128", name, (long long)N,
              (long long)K);
  QMM_REQUIRE(N * (K / kGroup) < (1ll << 30) && N <= static_cast<int64_t>(kMaxColBlocks) * kColsPerBlock,
              QMM_ERR_UNSUPPORTED, "%s: problem too large", name);
  QMM_REQUIRE(aligned(x, 16) && aligned(wq, 16) && aligned(scales, 16) && aligned(zeros, 16) &&
                  aligned(y, 4),
              QMM_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", name);
  return QMM_OK;
}

// ---------------------------------------------------------------------------
// Built-in scratch for callers that must not allocate.
//
// The array lives in the library's device image: every GPU that loads the
// library holds these bytes until the process exits.  On the host its name is
// only a handle, not an address a kernel can use; the device address is
// looked up once per device with cudaGetSymbolAddress while that device is
// current, and that pointer is what gets passed to the kernel.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = QMM_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void* g_static_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device (looked up on the
// first call per device, cached afterwards).
static int static_scratch_address(void** out) {
  int dev = -1;
  QMM_CUDA_TRY(cudaGetDevice(&dev));
  QMM_REQUIRE(dev >= 0 && dev < kMaxDevices, QMM_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    QMM_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    QMM_REQUIRE(p != nullptr && aligned(p, 256), QMM_ERR_CUDA,
                "cudaGetSymbolAddress returned an unusable address for the built-in scratch");
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return QMM_OK;
}

}  // namespace w4
}  // namespace qmm


extern "C" {

size_t qmm_w4a16_g128_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  using namespace qmm::w4;
  if (M < 1 || N < 128 || K < kGroup || N % 128 || K % kGroup) return 0;
  if (M > kDecodeMaxM) return 0;  // the prefill GEMM needs no scratch
  const int G = static_cast<int>(K / kGroup);
  const int C = col_blocks(N);
  const int U = G * C;
  const int P = grid_size(U, static_cast<int>(M));
  const int slots = slots_for(G, U, P);
  const size_t counters = counter_bytes(C);
  return counters + static_cast<size_t>(C) * slots * rows_padded(static_cast<int>(M)) * kColsPerBlock *
                        sizeof(float);
}

int qmm_w4a16_g128(const uint16_t* x, const uint8_t* wq, const uint16_t* scales,
                   const uint8_t* zeros, int zeros_packed, uint16_t* y, int64_t M, int64_t N,
                   int64_t K, int64_t group, void* workspace, size_t workspace_bytes,
                   unsigned flags, void* stream) {
  using namespace qmm;
  using namespace qmm::w4;
  if (int rc = check_args("qmm_w4a16_g128", x, wq, scales, zeros, y, M, N, K, group, (1ll << 30) - 1)) return rc;
  if (M > kDecodeMaxM) {
    // prefill-sized M: the tcgen05 GEMM with the nibbles dequantised in shared memory (no scratch)
    if (int st = read_device_status())
      return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
    return w4a16_tcgen05(x, wq, scales, zeros, zeros_packed, y, M, N, K, 0u, static_cast<cudaStream_t>(stream));
  }
  const size_t need = qmm_w4a16_g128_workspace_bytes(M, N, K);
  QMM_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned(workspace, 256),
              QMM_ERR_WORKSPACE, "qmm_w4a16_g128: workspace of %zu bytes (256-byte aligned) required",
              need);
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  return run("qmm_w4a16_g128", x, wq, scales, zeros, zeros_packed, y, M, N, K, workspace, flags,
             device_status_word(), static_cast<cudaStream_t>(stream));
}

// qmm_w4a16_g128 for callers that cannot allocate: the split-K scratch is the
// library's own fixed array instead of a caller-provided workspace.
//
// Nothing here calls cudaMalloc, cudaFree, a host allocator of the CUDA
// runtime or any library routine that allocates.  The first call on a device
// looks up the array's device address (cudaGetSymbolAddress, with that device
// current); make that first call outside any stream capture.  The arrival
// counters at the head of the array are cleared on the stream before every
// launch, so a call never depends on what an earlier call (possibly one that
// was cut short) left behind; the partial tiles behind them are overwritten
// before they are read.  All calls on a device share the one array: two calls
// that can overlap on the GPU (different streams without an ordering between
// them) race on it and must be serialised by the caller.
int qmm_w4a16_g128_static_scratch(const uint16_t* x, const uint8_t* wq, const uint16_t* scales,
                                  const uint8_t* zeros, int zeros_packed, uint16_t* y, int64_t M,
                                  int64_t N, int64_t K, int64_t group, void* stream) {
  using namespace qmm;
  using namespace qmm::w4;
  if (int rc = check_args("qmm_w4a16_g128_static_scratch", x, wq, scales, zeros, y, M, N, K, group, kDecodeMaxM))
    return rc;
  const size_t need = qmm_w4a16_g128_workspace_bytes(M, N, K);
  QMM_REQUIRE(need > 0 && need <= kStaticScratchBytes, QMM_ERR_WORKSPACE,
              "qmm_w4a16_g128_static_scratch: this shape needs %zu bytes of scratch but the built-in "
              "array holds %zu; use qmm_w4a16_g128 with a caller-provided workspace",
              need, kStaticScratchBytes);
  // The library's status word (where a device-side wait that gives up is
  // recorded) is pinned host memory created on first use by any other entry
  // point or by qmm_device_status().  This call will not create it, because
  // that allocates; when it exists it is honoured as everywhere else.
  if (int st = read_device_status_if_ready())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  QMM_CUDA_TRY(cudaMemsetAsync(scratch, 0, counter_bytes(col_blocks(N)), st));
  return run("qmm_w4a16_g128_static_scratch", x, wq, scales, zeros, zeros_packed, y, M, N, K, scratch,
             0u, device_status_word_if_ready(), st);
}

}  // extern "C"
