// int4 group-wise (g128, asymmetric) weight-only matmul at decode sizes (M <= 32).
//
//   y[M,N] = bf16( x[M,K] @ ((q[K,N] - z[K/128,N]) * s[K/128,N]) )
//
// HBM-bound: the packed weights (K*N/2 bytes) are read exactly once.  The work
// is cut into units of one 128-column block x one 128-k group (a 64-row x
// 128-byte tile, 8 KB); consecutive units are dealt evenly to a grid of
// resident CTAs (2 per SM), so every SM streams the same number of bytes.
//
// Per CTA: a producer warp issues TMA loads (packed weights with the 128-byte
// swizzle, scales and zero points as bulk copies) into an 8-deep ring and
// stages the activations of the group (k-permuted to match the MMA fragment,
// plus the per-row group sums); eight consumer warps each own 16 columns.
// A consumer reads the tile with ldmatrix.trans, turns nibbles into bf16
// (128 + q) with one logic op each, and feeds mma.sync.m16n8k16 with the
// weights as the 16-row operand and the activations as the 8-column operand.
// Per group the accumulator is corrected and scaled:
//   y += s[g,n] * (acc - (128 + z[g,n]) * sum_k x[m,k])
// Partial sums of CTAs sharing a column block meet in the caller's workspace;
// the last CTA to arrive adds them in a fixed order (deterministic result) and
// writes bf16.  The workspace counters are left at zero.
#include <mutex>

#include "common.cuh"

namespace qmm {
namespace w4 {

constexpr int kColsPerBlock = 128;   // columns per unit (= bytes per TMA row)
constexpr int kGroup = 128;          // k per unit
constexpr int kRowsPerUnit = 64;     // packed byte-rows per unit
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kXRowBytes = 288;      // 128 bf16 + 32 B pad: conflict-free 8-byte fragment reads

template <int MT>
struct Smem {
  static constexpr int kW = kRowsPerUnit * kColsPerBlock;  // 8192
  static constexpr int kS = kColsPerBlock * 2;             // 256
  static constexpr int kZ = kColsPerBlock;                 // 128 (64 used when packed)
  static constexpr int kSx = 128;                          // MT*8 floats, padded
  static constexpr int kX = MT * 8 * kXRowBytes;
  static constexpr int kOffS = kW;
  static constexpr int kOffZ = kOffS + kS;
  static constexpr int kOffSx = kOffZ + kZ;
  static constexpr int kOffX = kOffSx + kSx;
  static constexpr int kStage = ((kOffX + kX + 1023) / 1024) * 1024;
  static constexpr int kStages = (MT <= 2) ? 8 : 6;
  static constexpr int kBarBytes = 1024;
  static constexpr int kTotal = kStages * kStage + kBarBytes + 1024;  // + alignment slack
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

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// CTA that owns unit u when U units are dealt to P CTAs as [i*U/P, (i+1)*U/P).
__device__ __forceinline__ int cta_of_unit(long long u, int P, int U) {
  return static_cast<int>(((u + 1) * P - 1) / U);
}

template <int MT, bool ZP_PACKED>
__global__ void __launch_bounds__(kThreads, 2)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap wmap, const uint16_t* __restrict__ x,
                    const uint16_t* __restrict__ scales, const uint8_t* __restrict__ zeros,
                    uint16_t* __restrict__ y, float* __restrict__ ws_partial,
                    int* __restrict__ ws_counter, int M, int N, int K, int G, int U, int max_slots,
                    int* status) {
  using L = Smem<MT>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * L::kStage);
  uint64_t* empty = full + S;
  uint64_t* sync_bar = empty + S;  // consumer-only rendezvous with a bounded wait
  int* flag = reinterpret_cast<int*>(sync_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int P = gridDim.x;
  const int u_begin = static_cast<int>((static_cast<long long>(blockIdx.x) * U) / P);
  const int u_end = static_cast<int>((static_cast<long long>(blockIdx.x + 1) * U) / P);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      dev::mbar_init(&full[s], 2);                // TMA transaction arrive + activation staging
      dev::mbar_init(&empty[s], kConsumerWarps);  // one arrive per consumer warp
    }
    dev::mbar_init(sync_bar, kConsumerWarps);
    dev::fence_mbar_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) dev::tma_prefetch_desc(&wmap);
    const uint64_t policy = dev::policy_evict_first();
    constexpr int kPasses = MT * 4;  // a pass = 2 rows x 16 lanes x 16 bytes
    uint4 xr[kPasses];
    auto load_x = [&](int u) {
      const int g = u % G;
#pragma unroll
      for (int p = 0; p < kPasses; ++p) {
        const int row = p * 2 + (lane >> 4);
        if (row < M) {
          const uint16_t* src = x + static_cast<size_t>(row) * K + g * kGroup + (lane & 15) * 8;
          xr[p] = __ldg(reinterpret_cast<const uint4*>(src));
        } else {
          xr[p] = make_uint4(0, 0, 0, 0);
        }
      }
    };
    if (u_begin < u_end) load_x(u_begin);
    int it = 0;
    for (int u = u_begin; u < u_end; ++u, ++it) {
      const int s = it % S;
      const uint32_t ph = (it / S) & 1;
      if (!dev::mbar_wait(&empty[s], ph ^ 1, status, 1)) break;
      uint8_t* st = smem + s * L::kStage;
      const int c = u / G, g = u % G;
      if (lane == 0) {
        const uint32_t zbytes = ZP_PACKED ? 64 : 128;
        dev::mbar_expect_tx(&full[s], L::kW + L::kS + zbytes);
        dev::tma_load_2d_hint(st, &wmap, &full[s], c * kColsPerBlock, g * kRowsPerUnit, policy);
        bulk_copy_g2s(st + L::kOffS, scales + static_cast<size_t>(g) * N + c * kColsPerBlock,
                      L::kS, &full[s]);
        const uint8_t* zsrc = ZP_PACKED
                                  ? zeros + static_cast<size_t>(g) * (N / 2) + c * (kColsPerBlock / 2)
                                  : zeros + static_cast<size_t>(g) * N + c * kColsPerBlock;
        bulk_copy_g2s(st + L::kOffZ, zsrc, zbytes, &full[s]);
      }
      // activations of this group: permute every 4 consecutive k from (0,1,2,3)
      // to (0,2,1,3) and sum each row over the group
      float* sx = reinterpret_cast<float*>(st + L::kOffSx);
#pragma unroll
      for (int p = 0; p < kPasses; ++p) {
        const int row = p * 2 + (lane >> 4);
        const uint4 v = xr[p];
        uint4 o;
        o.x = __byte_perm(v.x, v.y, 0x5410);
        o.y = __byte_perm(v.x, v.y, 0x7632);
        o.z = __byte_perm(v.z, v.w, 0x5410);
        o.w = __byte_perm(v.z, v.w, 0x7632);
        *reinterpret_cast<uint4*>(st + L::kOffX + row * kXRowBytes + (lane & 15) * 16) = o;
        float sum = __uint_as_float(v.x << 16) + __uint_as_float(v.x & 0xFFFF0000u) +
                    __uint_as_float(v.y << 16) + __uint_as_float(v.y & 0xFFFF0000u) +
                    __uint_as_float(v.z << 16) + __uint_as_float(v.z & 0xFFFF0000u) +
                    __uint_as_float(v.w << 16) + __uint_as_float(v.w & 0xFFFF0000u);
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        if ((lane & 15) == 0) sx[row] = sum;
      }
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(&full[s]);
      if (u + 1 < u_end) load_x(u + 1);
    }
  } else {
    // ------------------------------ consumers -----------------------------
    const int g8 = lane >> 2;  // 0..7
    const int t4 = lane & 3;   // 0..3
    const int ctid = threadIdx.x;  // 0..255
    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;

    uint32_t sync_phase = 0;
    // Rendezvous of the eight consumer warps.  An mbarrier with a bounded wait
    // rather than bar.sync, so that a warp that gave up earlier cannot leave
    // the others waiting for ever.
    auto consumer_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(sync_bar);
      const bool r = dev::mbar_wait(sync_bar, sync_phase, status, 3);
      sync_phase ^= 1;
      __syncwarp();
      return r;
    };
    auto flush = [&](int c) {
      const int first = cta_of_unit(static_cast<long long>(c) * G, P, U);
      const int last = cta_of_unit(static_cast<long long>(c) * G + G - 1, P, U);
      const int nslots = last - first + 1;
      const int col = c * kColsPerBlock + warp * 16 + 2 * g8;
      if (nslots == 1) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int m = mt * 8 + 2 * t4 + r;
            if (m < M)
              *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(m) * N + col) =
                  dev::pack_bf16x2(yacc[mt][r], yacc[mt][2 + r]);
          }
        return;
      }
      const int slot = static_cast<int>(blockIdx.x) - first;
      float* part = ws_partial + (static_cast<size_t>(c) * max_slots + slot) * (MT * 8) * kColsPerBlock;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int m = mt * 8 + 2 * t4 + r;
          if (m < M)
            __stcg(reinterpret_cast<float2*>(part + m * kColsPerBlock + warp * 16 + 2 * g8),
                   make_float2(yacc[mt][r], yacc[mt][2 + r]));
        }
      __threadfence();
      if (!consumer_sync()) return;
      if (ctid == 0) {
        const int old = atomicAdd(&ws_counter[c], 1);
        *reinterpret_cast<volatile int*>(flag) = (old + 1 == nslots) ? 1 : 0;
      }
      if (!consumer_sync()) return;
      const bool is_last = (*reinterpret_cast<volatile int*>(flag) != 0);
      if (is_last) {
        __threadfence();
        const float* base = ws_partial + static_cast<size_t>(c) * max_slots * (MT * 8) * kColsPerBlock;
        for (int idx = ctid; idx < M * (kColsPerBlock / 2); idx += 256) {
          const int m = idx / (kColsPerBlock / 2);
          const int cp = (idx % (kColsPerBlock / 2)) * 2;
          float a = 0.f, b = 0.f;
          for (int sl = 0; sl < nslots; ++sl) {
            const float2 v = __ldcg(reinterpret_cast<const float2*>(
                base + (static_cast<size_t>(sl) * (MT * 8) + m) * kColsPerBlock + cp));
            a += v.x;
            b += v.y;
          }
          *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(m) * N + c * kColsPerBlock + cp) =
              dev::pack_bf16x2(a, b);
        }
        if (ctid == 0) ws_counter[c] = 0;
      }
      // the flag word is reused by the next flush of this CTA
      consumer_sync();
    };

    int cur_c = (u_begin < u_end) ? u_begin / G : 0;
    int it = 0;
    bool ok = true;
    for (int u = u_begin; u < u_end; ++u, ++it) {
      const int s = it % S;
      const uint32_t ph = (it / S) & 1;
      const int c = u / G;
      if (c != cur_c) {
        flush(cur_c);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;
        cur_c = c;
      }
      if (!dev::mbar_wait(&full[s], ph, status, 2)) {
        ok = false;
        break;
      }
      const uint8_t* st = smem + s * L::kStage;
      const uint32_t st_addr = dev::smem_u32(st);
      float acc[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // four 8-row matrices: rows 32h + 8j + (lane % 8), this warp's 16-byte chunk
        const int row = 32 * h + lane;
        uint32_t wreg[4];
        ldmatrix_x4_trans(st_addr + row * 128 + ((warp ^ (row & 7)) << 4), wreg);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w = wreg[j];
          const uint32_t r0 = (w & 0x000F000Fu) | 0x43004300u;          // col 2g,   k 4t, 4t+2
          const uint32_t r1 = ((w >> 4) & 0x000F000Fu) | 0x43004300u;   // col 2g,   k 4t+1, 4t+3
          const uint32_t r2 = ((w >> 8) & 0x000F000Fu) | 0x43004300u;   // col 2g+1, k 4t, 4t+2
          const uint32_t r3 = ((w >> 12) & 0x000F000Fu) | 0x43004300u;  // col 2g+1, k 4t+1, 4t+3
          const int slab = 4 * h + j;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint2 xf = *reinterpret_cast<const uint2*>(
                st + L::kOffX + (mt * 8 + g8) * kXRowBytes + slab * 32 + t4 * 8);
            mma_bf16_16816(acc[mt], r0, r2, r1, r3, xf.x, xf.y);
          }
        }
      }
      // group epilogue: this thread holds columns (2g, 2g+1) of its warp's
      // chunk for rows (2t, 2t+1) of each 8-row tile
      const int lc = warp * 16 + 2 * g8;
      const uint32_t s2 = *reinterpret_cast<const uint32_t*>(st + L::kOffS + lc * 2);
      const float sc0 = __uint_as_float(s2 << 16);
      const float sc1 = __uint_as_float(s2 & 0xFFFF0000u);
      float z0, z1;
      if (ZP_PACKED) {
        const uint32_t zb = st[L::kOffZ + (lc >> 1)];
        z0 = static_cast<float>(zb & 0xF);
        z1 = static_cast<float>(zb >> 4);
      } else {
        const uint32_t zb = *reinterpret_cast<const uint16_t*>(st + L::kOffZ + lc);
        z0 = static_cast<float>(zb & 0xFF);
        z1 = static_cast<float>(zb >> 8);
      }
      const float off0 = -(128.f + z0), off1 = -(128.f + z1);
      const float* sx = reinterpret_cast<const float*>(st + L::kOffSx);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float2 sxm = *reinterpret_cast<const float2*>(sx + mt * 8 + 2 * t4);
        yacc[mt][0] = fmaf(sc0, fmaf(off0, sxm.x, acc[mt][0]), yacc[mt][0]);
        yacc[mt][1] = fmaf(sc0, fmaf(off0, sxm.y, acc[mt][1]), yacc[mt][1]);
        yacc[mt][2] = fmaf(sc1, fmaf(off1, sxm.x, acc[mt][2]), yacc[mt][2]);
        yacc[mt][3] = fmaf(sc1, fmaf(off1, sxm.y, acc[mt][3]), yacc[mt][3]);
      }
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(&empty[s]);
    }
    if (ok && u_begin < u_end) flush(cur_c);
  }
}

template <int MT, bool ZP>
static int launch(const CUtensorMap& wmap, const uint16_t* x, const uint16_t* scales,
                  const uint8_t* zeros, uint16_t* y, float* ws_partial, int* ws_counter, int M, int N,
                  int K, int G, int U, int P, int max_slots, cudaStream_t stream) {
  using L = Smem<MT>;
  static bool configured = false;
  auto kern = w4a16_decode_kernel<MT, ZP>;
  if (!configured) {
    QMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  kern<<<P, kThreads, L::kTotal, stream>>>(wmap, x, scales, zeros, y, ws_partial, ws_counter, M, N,
                                           K, G, U, max_slots, device_status_word());
  QMM_CHECK_LAUNCH("w4a16_decode_kernel");
  return QMM_OK;
}

static int grid_size(int U) {
  // two resident CTAs per SM; small problems get at least two units per CTA so
  // that few CTAs share a column block
  const int p = 2 * num_sms();
  const int q = (U + 1) / 2;
  return q < p ? q : p;
}
static int slots_for(int G, int U, int P) {
  // a column block of G units is shared by at most ceil(G*P/U) + 1 CTAs
  return static_cast<int>((static_cast<long long>(G) * P + U - 1) / U) + 1;
}
static int rows_padded(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : 32); }

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

constexpr int kMaxDevices = 64;
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

// Same launch as launch<MT, ZP>() but with the status pointer supplied by the
// caller instead of created on demand (creating it would allocate).
template <int MT, bool ZP>
static int launch_no_alloc(const CUtensorMap& wmap, const uint16_t* x, const uint16_t* scales,
                           const uint8_t* zeros, uint16_t* y, float* ws_partial, int* ws_counter,
                           int M, int N, int K, int G, int U, int P, int max_slots, int* status,
                           cudaStream_t stream) {
  using L = Smem<MT>;
  static bool configured = false;
  auto kern = w4a16_decode_kernel<MT, ZP>;
  if (!configured) {
    QMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  kern<<<P, kThreads, L::kTotal, stream>>>(wmap, x, scales, zeros, y, ws_partial, ws_counter, M, N,
                                           K, G, U, max_slots, status);
  QMM_CHECK_LAUNCH("w4a16_decode_kernel");
  return QMM_OK;
}

}  // namespace w4
}  // namespace qmm

extern "C" {

size_t qmm_w4a16_g128_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  using namespace qmm::w4;
  if (M < 1 || M > 32 || N < kColsPerBlock || K < kGroup || N % kColsPerBlock || K % kGroup) return 0;
  const int G = static_cast<int>(K / kGroup);
  const int C = static_cast<int>(N / kColsPerBlock);
  const int U = G * C;
  const int P = grid_size(U);
  const int slots = slots_for(G, U, P);
  const size_t counters = (static_cast<size_t>(C) * sizeof(int) + 255) / 256 * 256;
  return counters + static_cast<size_t>(C) * slots * rows_padded(static_cast<int>(M)) * kColsPerBlock *
                        sizeof(float);
}

int qmm_w4a16_g128(const uint16_t* x, const uint8_t* wq, const uint16_t* scales,
                   const uint8_t* zeros, int zeros_packed, uint16_t* y, int64_t M, int64_t N,
                   int64_t K, int64_t group, void* workspace, size_t workspace_bytes,
                   void* stream) {
  using namespace qmm;
  using namespace qmm::w4;
  QMM_REQUIRE(x && wq && scales && zeros && y, QMM_ERR_INVALID_ARGUMENT,
              "qmm_w4a16_g128: null tensor pointer");
  QMM_REQUIRE(group == kGroup, QMM_ERR_UNSUPPORTED, "qmm_w4a16_g128: group must be 128, got %lld",
              (long long)group);
  QMM_REQUIRE(M >= 1 && M <= 32, QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128: decode kernel covers 1 <= M <= 32, got %lld", (long long)M);
  QMM_REQUIRE(N >= kColsPerBlock && N % kColsPerBlock == 0 && K >= kGroup && K % kGroup == 0,
              QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128: N (%lld) and K (%lld) must be positive multiples of 128", (long long)N,
              (long long)K);
  QMM_REQUIRE(N * (K / kGroup) < (1ll << 30), QMM_ERR_UNSUPPORTED, "qmm_w4a16_g128: problem too large");
  QMM_REQUIRE(aligned(x, 16) && aligned(wq, 16) && aligned(scales, 16) && aligned(zeros, 16) &&
                  aligned(y, 4),
              QMM_ERR_INVALID_ARGUMENT, "qmm_w4a16_g128: tensors must be 16-byte aligned");
  const size_t need = qmm_w4a16_g128_workspace_bytes(M, N, K);
  QMM_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned(workspace, 256),
              QMM_ERR_WORKSPACE, "qmm_w4a16_g128: workspace of %zu bytes (256-byte aligned) required",
              need);
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);

  const int G = static_cast<int>(K / kGroup);
  const int C = static_cast<int>(N / kColsPerBlock);
  const int U = G * C;
  const int P = grid_size(U);
  const int slots = slots_for(G, U, P);
  const size_t counters = (static_cast<size_t>(C) * sizeof(int) + 255) / 256 * 256;
  int* ws_counter = static_cast<int*>(workspace);
  float* ws_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counters);

  CUtensorMap wmap;
  if (int rc = make_tensor_map_2d(&wmap, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                                  static_cast<uint64_t>(K / 2), static_cast<uint64_t>(N),
                                  static_cast<uint64_t>(N), kRowsPerUnit, kColsPerBlock,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
#define QMM_W4_LAUNCH(MT)                                                                        \
  (zeros_packed ? launch<MT, true>(wmap, x, scales, zeros, y, ws_partial, ws_counter, m, n, k, G, \
                                   U, P, slots, st)                                              \
                : launch<MT, false>(wmap, x, scales, zeros, y, ws_partial, ws_counter, m, n, k,  \
                                    G, U, P, slots, st))
  if (M <= 8) return QMM_W4_LAUNCH(1);
  if (M <= 16) return QMM_W4_LAUNCH(2);
  return QMM_W4_LAUNCH(4);
#undef QMM_W4_LAUNCH
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
  QMM_REQUIRE(x && wq && scales && zeros && y, QMM_ERR_INVALID_ARGUMENT,
              "qmm_w4a16_g128_static_scratch: null tensor pointer");
  QMM_REQUIRE(group == kGroup, QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128_static_scratch: group must be 128, got %lld", (long long)group);
  QMM_REQUIRE(M >= 1 && M <= 32, QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128_static_scratch: covers 1 <= M <= 32, got %lld", (long long)M);
  QMM_REQUIRE(N >= kColsPerBlock && N % kColsPerBlock == 0 && K >= kGroup && K % kGroup == 0,
              QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128_static_scratch: N (%lld) and K (%lld) must be positive multiples of 128",
              (long long)N, (long long)K);
  QMM_REQUIRE(N * (K / kGroup) < (1ll << 30), QMM_ERR_UNSUPPORTED,
              "qmm_w4a16_g128_static_scratch: problem too large");
  QMM_REQUIRE(aligned(x, 16) && aligned(wq, 16) && aligned(scales, 16) && aligned(zeros, 16) &&
                  aligned(y, 4),
              QMM_ERR_INVALID_ARGUMENT,
              "qmm_w4a16_g128_static_scratch: tensors must be 16-byte aligned");
  const size_t need = qmm_w4a16_g128_workspace_bytes(M, N, K);
  QMM_REQUIRE(need > 0 && need <= kStaticScratchBytes, QMM_ERR_WORKSPACE,
              "qmm_w4a16_g128_static_scratch: this shape needs %zu bytes of scratch but the built-in "
              "array holds %zu; use qmm_w4a16_g128 with a caller-provided workspace",
              need, kStaticScratchBytes);
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;

  const int G = static_cast<int>(K / kGroup);
  const int C = static_cast<int>(N / kColsPerBlock);
  const int U = G * C;
  const int P = grid_size(U);
  const int slots = slots_for(G, U, P);
  const size_t counters = (static_cast<size_t>(C) * sizeof(int) + 255) / 256 * 256;
  int* ws_counter = static_cast<int*>(scratch);
  float* ws_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + counters);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  QMM_CUDA_TRY(cudaMemsetAsync(ws_counter, 0, counters, st));

  CUtensorMap wmap;
  if (int rc = make_tensor_map_2d(&wmap, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                                  static_cast<uint64_t>(K / 2), static_cast<uint64_t>(N),
                                  static_cast<uint64_t>(N), kRowsPerUnit, kColsPerBlock,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // A wait that gives up is reported through the library's status word when
  // that word exists already (any other entry point, or qmm_device_status(),
  // creates it); this call will not create it, because that allocates.
  int* status = device_status_word_if_ready();
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
#define QMM_W4_LAUNCH_NA(MT)                                                                       \
  (zeros_packed ? launch_no_alloc<MT, true>(wmap, x, scales, zeros, y, ws_partial, ws_counter, m, \
                                            n, k, G, U, P, slots, status, st)                     \
                : launch_no_alloc<MT, false>(wmap, x, scales, zeros, y, ws_partial, ws_counter, m, \
                                             n, k, G, U, P, slots, status, st))
  if (M <= 8) return QMM_W4_LAUNCH_NA(1);
  if (M <= 16) return QMM_W4_LAUNCH_NA(2);
  return QMM_W4_LAUNCH_NA(4);
#undef QMM_W4_LAUNCH_NA
}

}  // extern "C"
