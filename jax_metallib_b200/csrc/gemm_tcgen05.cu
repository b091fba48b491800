// tcgen05 / TMEM GEMMs for the prefill-sized quantized matmuls (sm_100a).
//
// Two kernels share one skeleton: a persistent CTA per SM walks output tiles;
// warp 0 feeds shared memory with TMA (128-byte swizzle), one thread of warp 1
// issues tcgen05.mma into a double-buffered TMEM accumulator (2 x 256 columns),
// warps 2-5 drain the accumulator with tcgen05.ld and apply the fused epilogue
// while the next tile's MMAs run.  Every wait is bounded.
//
//  (1) i8gemm: acc[M,N] = a[M,K] . b[K,N], int8/uint8 operands, int32
//      accumulate (kind::i8, exact).  a is K-major, b is consumed N-major
//      straight from its row-major [K,N] layout (MN-major descriptor), so no
//      transposed copy of b is ever made.  Tile 128 (m) x 256 (n) x 128 (k).
//      Epilogue: optional int32 store and/or float(acc) * row[m] * col[n].
//
//  (2) w8a16: y[M,N] = bf16((x[M,K] @ float(w[K,N])) * scale[N]), bf16
//      activations, int8 weights.  The weight tile is the 128-row MMA operand
//      (MN-major: its 128 output channels are contiguous in memory), the
//      activation tile the 256-column operand, so each CTA converts only
//      128 x 64 weights per k-step: converter warps read the raw int8 tile,
//      turn it into bf16 (exactly) and write the MMA's swizzled layout.  The
//      accumulator holds the transposed tile (lane = output channel), so the
//      per-channel scale is one register per thread and stores of a warp are
//      contiguous along N.  Tile 128 (n) x 256 (m) x 64 (k).
#include "common.cuh"

namespace qmm {
namespace tc {

constexpr int kEpiWarps = 4;
constexpr uint32_t kSwizzle128 = 2;  // UMMA layout type of the 128-byte swizzle

// ============================================================================
// (1) int8 x int8 -> int32
// ============================================================================
namespace i8 {
constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK;       // 16 KB
constexpr int kBBytes = BK * BN;       // 32 KB: two [BK x 128] column blocks
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment*/;

__global__ void __launch_bounds__(kThreads, 1)
i8gemm_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
              int32_t* __restrict__ acc_out, float* __restrict__ f_out,
              const float* __restrict__ row_scale, const float* __restrict__ col_scale, int M, int N,
              int K, uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;   // accumulator ready for the epilogue
  uint64_t* tempty = tfull + 2;        // accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      dev::mbar_init(&full[s], 1);
      dev::mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      dev::mbar_init(&tfull[i], 1);
      dev::mbar_init(&tempty[i], kEpiWarps);
    }
    dev::fence_mbar_init();
  }
  if (warp == 1) {
    dev::tmem_alloc(tmem_slot, 512);
    dev::tmem_relinquish();
  }
  dev::tc_fence_before();
  __syncthreads();
  dev::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      dev::tma_prefetch_desc(&amap);
      dev::tma_prefetch_desc(&bmap);
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!dev::mbar_wait(&empty[s], ph ^ 1, status, 11)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          dev::mbar_expect_tx(&full[s], kStageBytes);
          dev::tma_load_2d(st, &amap, &full[s], kb * BK, tm * BM);
          dev::tma_load_2d(st + kABytes, &bmap, &full[s], tn * BN, kb * BK);
          dev::tma_load_2d(st + kABytes + BK * 128, &bmap, &full[s], tn * BN + 128, kb * BK);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer -----------------------------
    if (lane == 0) {
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int as = tcount & 1;
        if (!dev::mbar_wait(&tempty[as], ((tcount >> 1) & 1) ^ 1, status, 12)) { ok = false; break; }
        dev::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!dev::mbar_wait(&full[s], ph, status, 13)) { ok = false; break; }
          dev::tc_fence_after();
          const uint32_t a_addr = dev::smem_u32(smem + s * kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // a: K-major, 32 bytes of k per instruction inside the 128-byte swizzle span
            const uint64_t adesc = dev::make_smem_desc(a_addr + k * 32, 16, 1024, kSwizzle128);
            // b: MN-major, 32 k-rows (4 KB) per instruction; column blocks 16 KB apart
            const uint64_t bdesc =
                dev::make_smem_desc(b_addr + k * 32 * 128, BK * 128, 1024, kSwizzle128);
            dev::umma_i8(d_tmem, adesc, bdesc, idesc, (kb | k) != 0);
          }
          dev::tc_commit(&empty[s]);
        }
        if (ok) dev::tc_commit(&tfull[as]);
      }
    }
  } else {
    // ------------------------------ epilogue -------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int as = tcount & 1;
      if (!dev::mbar_wait(&tfull[as], (tcount >> 1) & 1, status, 14)) break;
      dev::tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const float rs = (f_out && row < M) ? __ldg(row_scale + row) : 0.f;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        dev::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BN + ch * 32, r);
        dev::tc_wait_ld();
        const int col0 = tn * BN + ch * 32;
        if (row < M) {
          if (acc_out) {
            int32_t* dst = acc_out + static_cast<size_t>(row) * N + col0;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (col0 + 4 * i < N)
                *reinterpret_cast<uint4*>(dst + 4 * i) =
                    make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          }
          if (f_out) {
            float* dst = f_out + static_cast<size_t>(row) * N + col0;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (col0 + 4 * i < N) {
                const float4 cs = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + 4 * i));
                float4 o;
                o.x = static_cast<float>(static_cast<int32_t>(r[4 * i])) * rs * cs.x;
                o.y = static_cast<float>(static_cast<int32_t>(r[4 * i + 1])) * rs * cs.y;
                o.z = static_cast<float>(static_cast<int32_t>(r[4 * i + 2])) * rs * cs.z;
                o.w = static_cast<float>(static_cast<int32_t>(r[4 * i + 3])) * rs * cs.w;
                *reinterpret_cast<float4*>(dst + 4 * i) = o;
              }
          }
        }
      }
      dev::tc_fence_before();
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(&tempty[as]);
    }
  }
  dev::tc_fence_before();
  __syncthreads();
  if (warp == 1) dev::tmem_dealloc(tmem_base, 512);
}
}  // namespace i8

// ============================================================================
// (2) bf16 activations x int8 weights (per-output-channel scale) -> bf16
// ============================================================================
namespace w8 {
constexpr int BNW = 128;   // output channels per tile (MMA M)
constexpr int BMX = 256;   // activation rows per tile (MMA N)
constexpr int BK = 64;
constexpr int kStages = 4;     // TMA ring: raw weights + activations
constexpr int kCvtBufs = 2;    // converted-weight buffers between the converter warps and the MMA
constexpr int kCvtWarps = 8;
constexpr int kRawBytes = BK * BNW;        // 8 KB  int8 [k][n]
constexpr int kCvtBytes = BK * BNW * 2;    // 16 KB bf16, two 64-channel blocks of [k][128 B]
constexpr int kXBytes = BMX * BK * 2;      // 32 KB bf16 [m][k]
constexpr int kStageBytes = kRawBytes + kXBytes;  // 40 KB
constexpr int kCvtBase = kStages * kStageBytes;   // 160 KB
constexpr int kThreads = (2 + kEpiWarps + kCvtWarps) * 32;
constexpr int kSmemBytes = kCvtBase + kCvtBufs * kCvtBytes + 1024 + 1024;
constexpr int kPanelTiles = 8;  // activation tiles swept together so that they stay in L2

// Eight int8 (one 8-byte read) -> eight bf16, exactly: the byte, biased to
// unsigned, becomes the low mantissa bits of 2^23 (an f32 holding 2^23 + 128 + v),
// the constant is subtracted and pairs are packed with round-to-nearest (exact,
// |v| <= 128 fits bf16's 8 significant bits).  The MMA needs both operands in
// one 16-bit format (an f16 weight operand against bf16 activations raises an
// illegal-instruction error on sm_100a), so the weights follow the activations.
__device__ __forceinline__ uint4 convert8(const uint2& in) {
  const uint32_t w[2] = {in.x ^ 0x80808080u, in.y ^ 0x80808080u};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float f0 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7440)) - 8388736.f;
    const float f1 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7441)) - 8388736.f;
    const float f2 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7442)) - 8388736.f;
    const float f3 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7443)) - 8388736.f;
    o[2 * i] = dev::pack_bf16x2(f0, f1);
    o[2 * i + 1] = dev::pack_bf16x2(f2, f3);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Tile order: activation tiles are swept in panels of kPanelTiles; inside a
// panel the weight tile changes slowest, so the CTAs that run together share
// one panel of activations (it stays in L2) and a handful of weight tiles.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_panel = kPanelTiles * tiles_n;
  const int p = tile / per_panel, r = tile - p * per_panel;
  const int rows = min(kPanelTiles, tiles_m - p * kPanelTiles);  // the last panel may be short
  tn = r / rows;
  tm = p * kPanelTiles + r % rows;
}

__global__ void __launch_bounds__(kThreads, 1)
w8a16_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
             const float* __restrict__ scale, uint16_t* __restrict__ y, int M, int N, int K,
             long long ldy, uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kCvtBase + kCvtBufs * kCvtBytes);  // TMA landed
  uint64_t* empty = full + kStages;     // MMAs that read the stage's activations retired
  uint64_t* cfull = empty + kStages;    // weights converted
  uint64_t* cempty = cfull + kCvtBufs;  // MMAs that read the converted buffer retired
  uint64_t* tfull = cempty + kCvtBufs;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BNW - 1) / BNW, tiles_m = (M + BMX - 1) / BMX;
  const int num_tiles = tiles_n * tiles_m;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      dev::mbar_init(&full[s], 1);
      dev::mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < kCvtBufs; ++i) {
      dev::mbar_init(&cfull[i], kCvtWarps);
      dev::mbar_init(&cempty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      dev::mbar_init(&tfull[i], 1);
      dev::mbar_init(&tempty[i], kEpiWarps);
    }
    dev::fence_mbar_init();
  }
  if (warp == 1) {
    dev::tmem_alloc(tmem_slot, 512);
    dev::tmem_relinquish();
  }
  dev::tc_fence_before();
  __syncthreads();
  dev::tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      dev::tma_prefetch_desc(&wmap);
      dev::tma_prefetch_desc(&xmap);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!dev::mbar_wait(&empty[s], ph ^ 1, status, 21)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          dev::mbar_expect_tx(&full[s], kRawBytes + kXBytes);
          dev::tma_load_2d(st, &wmap, &full[s], tn * BNW, kb * BK);
          dev::tma_load_2d(st + kRawBytes, &xmap, &full[s], kb * BK, tm * BMX);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer -----------------------------
    if (lane == 0) {
      int s = 0, c = 0, tcount = 0;
      uint32_t ph = 0, cph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int as = tcount & 1;
        if (!dev::mbar_wait(&tempty[as], ((tcount >> 1) & 1) ^ 1, status, 22)) { ok = false; break; }
        dev::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BMX;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!dev::mbar_wait(&full[s], ph, status, 23) ||
              !dev::mbar_wait(&cfull[c], cph, status, 24)) { ok = false; break; }
          dev::tc_fence_after();
          const uint32_t w_addr = dev::smem_u32(smem + kCvtBase + c * kCvtBytes);
          const uint32_t x_addr = dev::smem_u32(smem + s * kStageBytes + kRawBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // weights: MN-major, 16 k-rows (2 KB) per instruction, 64-channel blocks 8 KB apart
            const uint64_t adesc =
                dev::make_smem_desc(w_addr + k * 16 * 128, BK * 128, 1024, kSwizzle128);
            // activations: K-major, 32 bytes of k per instruction
            const uint64_t bdesc = dev::make_smem_desc(x_addr + k * 32, 16, 1024, kSwizzle128);
            dev::umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0);
          }
          dev::tc_commit(&empty[s]);    // frees the TMA stage (raw weights were consumed earlier)
          dev::tc_commit(&cempty[c]);   // frees the converted buffer
          if (++s == kStages) { s = 0; ph ^= 1; }
          if (++c == kCvtBufs) { c = 0; cph ^= 1; }
        }
        if (ok) dev::tc_commit(&tfull[as]);
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------ epilogue -------------------------------
    const int q = warp & 3;
    int tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int as = tcount & 1;
      if (!dev::mbar_wait(&tfull[as], (tcount >> 1) & 1, status, 25)) break;
      dev::tc_fence_after();
      const int n = tn * BNW + q * 32 + lane;  // this thread's output channel
      const float sc = (n < N) ? __ldg(scale + n) : 0.f;
#pragma unroll 1
      for (int ch = 0; ch < BMX / 32; ++ch) {
        uint32_t r[32];
        dev::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BMX + ch * 32, r);
        dev::tc_wait_ld();
        const int m0 = tm * BMX + ch * 32;
        // pair neighbouring channels so that every lane stores 4 bytes: even
        // lanes write rows m0+2j, odd lanes rows m0+2j+1
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a = __uint_as_float(r[2 * j]) * sc;
          const float b = __uint_as_float(r[2 * j + 1]) * sc;
          const float send = (lane & 1) ? a : b;
          const float got = __shfl_xor_sync(0xFFFFFFFFu, send, 1);
          const int m = m0 + 2 * j + (lane & 1);
          const uint32_t packed = (lane & 1) ? dev::pack_bf16x2(got, b) : dev::pack_bf16x2(a, got);
          const int n_even = n & ~1;
          if (m < M && n_even < N)
            *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(m) * ldy + n_even) = packed;
        }
      }
      dev::tc_fence_before();
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(&tempty[as]);
    }
  } else {
    // ------------------------------ converters -----------------------------
    // A half-warp reads one 128-byte raw row, 8 bytes per lane (conflict-free
    // in any permutation); each lane writes the 16-byte bf16 chunk it made, so
    // a quarter-warp store covers the eight chunks of one 128-byte row of one
    // 64-channel block: conflict-free as well, with no divergence.
    const int cw = warp - (2 + kEpiWarps);  // 0..7
    const int piece = lane & 15;            // 8 channels: [8*piece, 8*piece+8)
    const int rsub = lane >> 4;             // row within a pair
    int s = 0, c = 0;
    uint32_t ph = 0, cph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!dev::mbar_wait(&full[s], ph, status, 26) ||
            !dev::mbar_wait(&cempty[c], cph ^ 1, status, 27)) { ok = false; break; }
        const uint8_t* raw = smem + s * kStageBytes;
        uint8_t* dst = smem + kCvtBase + c * kCvtBytes + (piece >> 3) * (BK * 128);
        uint2 in[BK / (2 * kCvtWarps)];
#pragma unroll
        for (int p = 0; p < BK / (2 * kCvtWarps); ++p) {
          const int r = (p * kCvtWarps + cw) * 2 + rsub;  // k-row 0..63
          in[p] = *reinterpret_cast<const uint2*>(raw + r * 128 + (((piece >> 1) ^ (r & 7)) << 4) +
                                                  ((piece & 1) << 3));
        }
#pragma unroll
        for (int p = 0; p < BK / (2 * kCvtWarps); ++p) {
          const int r = (p * kCvtWarps + cw) * 2 + rsub;
          *reinterpret_cast<uint4*>(dst + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) = convert8(in[p]);
        }
        dev::fence_proxy_async();
        __syncwarp();
        if (lane == 0) dev::mbar_arrive(&cfull[c]);
        if (++s == kStages) { s = 0; ph ^= 1; }
        if (++c == kCvtBufs) { c = 0; cph ^= 1; }
      }
    }
  }
  dev::tc_fence_before();
  __syncthreads();
  if (warp == 1) dev::tmem_dealloc(tmem_base, 512);
}
}  // namespace w8

}  // namespace tc
}  // namespace qmm

// ----------------------------------------------------------------------------
// Host entry points (the tensor-core route; callers fall back for other shapes)
// ----------------------------------------------------------------------------
namespace qmm {

int i8gemm_tcgen05(const void* a, const void* b, int32_t* acc, const float* row_scale,
                   const float* col_scale, float* out, int64_t M, int64_t N, int64_t K,
                   int a_unsigned, int b_unsigned, cudaStream_t stream) {
  using namespace tc::i8;
  CUtensorMap amap, bmap;
  if (int rc = make_tensor_map_2d(&amap, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M,
                                  (uint64_t)K, (uint64_t)K, BM, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&bmap, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K,
                                  (uint64_t)N, (uint64_t)N, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  static bool configured = false;
  if (!configured) {
    QMM_CUDA_TRY(cudaFuncSetAttribute(i8gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
    configured = true;
  }
  const uint32_t idesc = dev::make_idesc(/*c=s32*/ 2, a_unsigned ? 0 : 1, b_unsigned ? 0 : 1,
                                         /*a K-major*/ 0, /*b MN-major*/ 1, BM, BN);
  const int tiles = static_cast<int>(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
  const int grid = tiles < num_sms() ? tiles : num_sms();
  i8gemm_kernel<<<grid, kThreads, kSmemBytes, stream>>>(amap, bmap, acc, out, row_scale, col_scale,
                                                        (int)M, (int)N, (int)K, idesc,
                                                        device_status_word());
  QMM_CHECK_LAUNCH("i8gemm_kernel");
  return QMM_OK;
}

int w8a16_tcgen05(const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y, int64_t M,
                  int64_t N, int64_t K, int64_t ldy, cudaStream_t stream) {
  using namespace tc::w8;
  CUtensorMap wmap, xmap;
  if (int rc = make_tensor_map_2d(&wmap, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K,
                                  (uint64_t)N, (uint64_t)N, BK, BNW, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&xmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M,
                                  (uint64_t)K, (uint64_t)K * 2, BMX, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  static bool configured = false;
  if (!configured) {
    QMM_CUDA_TRY(cudaFuncSetAttribute(w8a16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
    configured = true;
  }
  // operand "a" of the MMA = weights (bf16, MN-major), "b" = activations (bf16, K-major)
  const uint32_t idesc = dev::make_idesc(/*c=f32*/ 1, /*bf16*/ 1, /*bf16*/ 1,
                                         /*a MN-major*/ 1, /*b K-major*/ 0, BNW, BMX);
  const int tiles = static_cast<int>(((N + BNW - 1) / BNW) * ((M + BMX - 1) / BMX));
  const int grid = tiles < num_sms() ? tiles : num_sms();
  w8a16_kernel<<<grid, kThreads, kSmemBytes, stream>>>(wmap, xmap, scale, y, (int)M, (int)N, (int)K,
                                                       (long long)ldy, idesc, device_status_word());
  QMM_CHECK_LAUNCH("w8a16_kernel");
  return QMM_OK;
}

}  // namespace qmm
