// tcgen05 / TMEM GEMMs for the prefill-sized quantized matmuls (sm_100a).
//
// Both kernels keep one persistent CTA per SM that walks output tiles, feed
// shared memory with TMA (128-byte swizzle), accumulate in all 512 TMEM columns
// (two 256-column accumulators, one MMA-issuing thread each: a single thread
// cannot issue tcgen05.mma fast enough to keep the tensor pipe busy) and drain
// the accumulators with tcgen05.ld into a fused epilogue.  Every wait is bounded.
//
//  (1) i8gemm: acc[M,N] = a[M,K] . b[K,N], int8/uint8 operands, int32
//      accumulate (kind::i8, exact).  a is K-major, b is consumed N-major
//      straight from its row-major [K,N] layout (MN-major descriptor), so no
//      transposed copy of b is ever made.  Tile 256 (m, two accumulators) x
//      256 (n) x 128 (k).  Warps: one TMA producer, two MMA issuers, eight
//      epilogue warps (optional int32 store and/or float(acc) * row[m] * col[n]).
//
//  (2) w8a16: y[M,N] = bf16((x[M,K] @ float(w[K,N])) * scale[N]), bf16
//      activations, int8 weights.  The weight tile is the 128-row MMA operand
//      (MN-major: its 128 output channels are contiguous in memory), the
//      activation tile the 256-column operand; a CTA runs two weight blocks
//      against one activation tile (256 channels x 256 rows).  Warps: a TMA
//      producer for activations, one for raw int8 weights, two MMA issuers and
//      24 worker warps in three groups that take every third 64-k stage: a
//      group reads the raw tile, converts it to bf16 (exactly) and writes the
//      MMA's swizzled layout; when a tile's stages are done the same 24 warps
//      drain its accumulators.  The accumulator holds the transposed tile
//      (lane = output channel), so the per-channel scale is one register per
//      thread.  Leftover tiles of the last round are cut into halves or
//      quarters.  The output may be stored with multimem.st to a multicast
//      address (one store reaches the same offset of every rank's buffer:
//      the all-gather of a column-sharded linear happens in the epilogue), and
//      the launch can signal its completion to every rank.
#include <cstdlib>

#include "common.cuh"

namespace qmm {
namespace tc {

constexpr uint32_t kSwizzle128 = 2;  // UMMA layout type of the 128-byte swizzle

// ============================================================================
// (1) int8 x int8 -> int32
// ============================================================================
namespace i8 {
constexpr int BMB = 128;            // rows per MMA (its M); a full tile has two such blocks
constexpr int BN = 256, BK = 128;
constexpr int kStages = 3;
constexpr int kABlock = BMB * BK;      // 16 KB: [128 rows][128 k]
constexpr int kABytes = 2 * kABlock;   // 32 KB: both row blocks
constexpr int kBBytes = BK * BN;       // 32 KB: two [128 k][128 n] column blocks
constexpr int kStageBytes = kABytes + kBBytes;  // 64 KB
constexpr int kEpiWarpsI = 8;
// Warp roles: 0 TMA, 1 MMA issue for row block 0, 2-9 epilogue, 10 MMA issue for row block 1.
constexpr int kSecondMmaWarp = 2 + kEpiWarpsI;
constexpr int kThreads = (kSecondMmaWarp + 1) * 32;
// One 32 x 32 chunk of 4-byte results per epilogue warp, 128-byte swizzled, for the TMA stores of a CTA's last
// item.  It lies in the first stage of the operand ring, which is idle by then; shared memory of its own would
// take the CTA past 196 KB, into the SM's largest shared-memory split, for 32 KB that the ring already has.
constexpr int kOutStage = 32 * 128;
constexpr int kOutBase = 0;
static_assert(kEpiWarpsI * kOutStage <= kStageBytes, "the result chunks must fit in one stage of the ring");
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment*/;
static_assert(BK == 128, "the issue loop is written out for four 32-byte k-steps");

// Item i of this CTA.  A tile is 256 rows x 256 columns: two row blocks against
// one column tile (a 128 x 256 tile needs 94 bytes per clock and SM from L2 at
// the int8 MMA rate, more than L2 delivers to all SMs at once; sharing the
// column tile between two accumulators needs 63).  When whole tiles would leave
// half of the SMs idle, row blocks are dealt out singly.
struct Work {
  int tm2, tn, h0, nh;
};
__device__ __forceinline__ bool get_work(int i, int tiles_m2, int tiles_n, int halves, int M, Work& w) {
  const int v = blockIdx.x + i * gridDim.x;
  const int total = tiles_m2 * tiles_n * (halves ? 2 : 1);
  if (v >= total) return false;
  const int tile = halves ? (v >> 1) : v;
  w.tm2 = tile % tiles_m2;
  w.tn = tile / tiles_m2;
  w.h0 = halves ? (v & 1) : 0;
  w.nh = halves ? 1 : 2;
  const int blocks_left = (M - w.tm2 * 2 * BMB + BMB - 1) / BMB - w.h0;
  w.nh = max(0, min(w.nh, blocks_left));
  return true;
}

__global__ void __launch_bounds__(kThreads, 1)
i8gemm_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
              const __grid_constant__ CUtensorMap accmap, const __grid_constant__ CUtensorMap outmap,
              int32_t* __restrict__ acc_out, float* __restrict__ f_out,
              const float* __restrict__ row_scale, const float* __restrict__ col_scale, int M, int N,
              int K, uint32_t idesc, int halves, int staged_store, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;    // count 2: one commit per issuing thread
  uint64_t* tfull = empty + kStages;   // accumulators ready for the epilogue (count 2)
  uint64_t* tempty = tfull + 1;        // accumulators drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m2 = (M + 2 * BMB - 1) / (2 * BMB), tiles_n = (N + BN - 1) / BN;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      dev::mbar_init(&full[s], 1);
      dev::mbar_init(&empty[s], 2);
    }
    dev::mbar_init(tfull, 2);
    dev::mbar_init(tempty, kEpiWarpsI);
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
      uint32_t s = 0, ph = 0;
      bool ok = true;
      Work w;
      for (int i = 0; ok && get_work(i, tiles_m2, tiles_n, halves, M, w); ++i) {
        if (w.nh == 0) continue;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!dev::mbar_wait(&empty[s], ph ^ 1, status, 11)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          dev::mbar_expect_tx(&full[s], w.nh * kABlock + kBBytes);
          for (int h = w.h0; h < w.h0 + w.nh; ++h)
            dev::tma_load_2d(st + h * kABlock, &amap, &full[s], kb * BK, (w.tm2 * 2 + h) * BMB);
          dev::tma_load_2d(st + kABytes, &bmap, &full[s], w.tn * BN, kb * BK);
          dev::tma_load_2d(st + kABytes + BK * 128, &bmap, &full[s], w.tn * BN + 128, kb * BK);
          ph ^= (s == kStages - 1);
          s = (s == kStages - 1) ? 0 : s + 1;
        }
      }
    }
  } else if (warp == 1 || warp == kSecondMmaWarp) {
    // ------------------------------ MMA issuers ----------------------------
    // Issuer j multiplies row block j of every item that has it into accumulator j.  The issuing
    // thread is the serial resource (a tcgen05.mma costs it ~85 cycles, a poll or a commit about
    // as much), so descriptors are advanced by adds on their low halves, the ring index by a
    // select, and an absent block is a predicated-off instruction, not a branch.
    if (lane == 0) {
      const int me = (warp == 1) ? 0 : 1;
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (kSwizzle128 << 29);  // SBO, version, swizzle
      // a: K-major, 32 bytes of k per instruction inside the 128-byte swizzle span
      const uint32_t a_lo0 = (((dev::smem_u32(smem) >> 4) & 0x3FFF) | ((16u >> 4) << 16)) + me * (kABlock >> 4);
      // b: MN-major, 32 k-rows (4 KB) per instruction; column blocks 16 KB apart
      const uint32_t b_lo0 = ((dev::smem_u32(smem + kABytes) >> 4) & 0x3FFF) | (((BK * 128u) >> 4) << 16);
      constexpr uint32_t kStageStep = kStageBytes >> 4, kAStepK = 32 >> 4, kBStepK = (32 * 128) >> 4;
      const uint32_t d_tmem = tmem_base + me * BN;
      uint32_t s = 0, ph = 0;
      int items = 0;
      bool ok = true;
      Work w;
      for (int i = 0; ok && get_work(i, tiles_m2, tiles_n, halves, M, w); ++i) {
        if (w.nh == 0) continue;
        if (!dev::mbar_wait(tempty, (items & 1) ^ 1, status, 12)) break;
        dev::tc_fence_after();
        const uint32_t mine = (me >= w.h0) && (me < w.h0 + w.nh);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!dev::mbar_wait(&full[s], ph, status, 13)) { ok = false; break; }
          dev::tc_fence_after();
          const uint32_t a_s = a_lo0 + s * kStageStep, b_s = b_lo0 + s * kStageStep;
          dev::umma_i8_lh_if(mine, d_tmem, a_s, kDescHi, b_s, kDescHi, idesc, kb != 0);
          dev::umma_i8_lh_if(mine, d_tmem, a_s + kAStepK, kDescHi, b_s + kBStepK, kDescHi, idesc, 1);
          dev::umma_i8_lh_if(mine, d_tmem, a_s + 2 * kAStepK, kDescHi, b_s + 2 * kBStepK, kDescHi, idesc, 1);
          dev::umma_i8_lh_if(mine, d_tmem, a_s + 3 * kAStepK, kDescHi, b_s + 3 * kBStepK, kDescHi, idesc, 1);
          dev::tc_commit(&empty[s]);  // second arrival: the other issuer
          ph ^= (s == kStages - 1);
          s = (s == kStages - 1) ? 0 : s + 1;
        }
        if (ok) dev::tc_commit(tfull);
        ++items;
      }
    }
  } else {
    // ------------------------------ epilogue -------------------------------
    const int q = warp & 3;         // TMEM lane quarter this warp may access
    const int j = (warp - 2) >> 2;  // accumulator (row block) of this warp
    const uint64_t store_policy = dev::policy_evict_first();
    int items = 0;
    Work w;
    for (int i = 0; get_work(i, tiles_m2, tiles_n, halves, M, w); ++i) {
      if (w.nh == 0) continue;
      if (!dev::mbar_wait_relaxed_warp(tfull, items & 1, status, 14)) break;
      dev::tc_fence_after();
      // A lane holds one row of a 32 x 32 chunk.  Stored straight from registers, a warp's 16-byte stores
      // would touch 32 different 128-byte lines per instruction; instead the chunk goes to shared memory
      // (row r at r * 128, 16-byte piece p at p ^ (r & 7): conflict-free) and one TMA store writes it out,
      // clipped to the tensor's bounds.
      // results of the CTA's last item leave through shared memory and TMA stores (the ring is idle: every load
      // has been consumed once the accumulators are complete); earlier items overlap their plain stores with the
      // loads of the next item, which the producer has already started into the ring
      Work w_next;
      const bool staged = staged_store && !get_work(i + 1, tiles_m2, tiles_n, halves, M, w_next);
      const int row0 = (w.tm2 * 2 + j) * BMB + q * 32;
      const int row = row0 + lane;
      const bool mine = (j >= w.h0) && (j < w.h0 + w.nh) && row < M;
      const float rs = (f_out && mine) ? __ldg(row_scale + row) : 0.f;
      uint8_t* stage = smem + kOutBase + (warp - 2) * kOutStage;
      uint8_t* my_row = stage + lane * 128;
      if (j >= w.h0 && j < w.h0 + w.nh && row0 < M) {
#pragma unroll 1
        for (int ch = 0; ch < BN / 32; ++ch) {
          const int col0 = w.tn * BN + ch * 32;
          if (col0 >= N) break;
          uint32_t r[32];
          dev::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + j * BN + ch * 32, r);
          dev::tc_wait_ld();
          if (!staged) {
            // straight from registers: 16-byte stores of 32 different rows per instruction
            if (mine) {
              if (acc_out) {
                int32_t* dst = acc_out + static_cast<size_t>(row) * N + col0;
#pragma unroll
                for (int i4 = 0; i4 < 8; ++i4)
                  if (col0 + 4 * i4 < N)
                    *reinterpret_cast<uint4*>(dst + 4 * i4) = make_uint4(r[4 * i4], r[4 * i4 + 1], r[4 * i4 + 2], r[4 * i4 + 3]);
              }
              if (f_out) {
                float* dst = f_out + static_cast<size_t>(row) * N + col0;
#pragma unroll
                for (int i4 = 0; i4 < 8; ++i4)
                  if (col0 + 4 * i4 < N) {
                    const float4 cs = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + 4 * i4));
                    float4 o;
                    o.x = static_cast<float>(static_cast<int32_t>(r[4 * i4])) * rs * cs.x;
                    o.y = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 1])) * rs * cs.y;
                    o.z = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 2])) * rs * cs.z;
                    o.w = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 3])) * rs * cs.w;
                    *reinterpret_cast<float4*>(dst + 4 * i4) = o;
                  }
              }
            }
            continue;
          }
          if (acc_out) {
            if (lane == 0) dev::tma_store_wait_read();   // the previous store has read the buffer
            __syncwarp();
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4)
              *reinterpret_cast<uint4*>(my_row + ((i4 ^ (lane & 7)) << 4)) =
                  make_uint4(r[4 * i4], r[4 * i4 + 1], r[4 * i4 + 2], r[4 * i4 + 3]);
            dev::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              dev::tma_store_2d_hint(&accmap, stage, col0, row0, store_policy);
              dev::tma_store_commit();
            }
          }
          if (f_out) {
            float4 o[8];
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
              if (col0 + 4 * i4 < N) cs = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + 4 * i4));
              o[i4].x = static_cast<float>(static_cast<int32_t>(r[4 * i4])) * rs * cs.x;
              o[i4].y = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 1])) * rs * cs.y;
              o[i4].z = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 2])) * rs * cs.z;
              o[i4].w = static_cast<float>(static_cast<int32_t>(r[4 * i4 + 3])) * rs * cs.w;
            }
            if (lane == 0) dev::tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) *reinterpret_cast<float4*>(my_row + ((i4 ^ (lane & 7)) << 4)) = o[i4];
            dev::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              dev::tma_store_2d_hint(&outmap, stage, col0, row0, store_policy);
              dev::tma_store_commit();
            }
          }
        }
      }
      dev::tc_fence_before();
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(tempty);
      ++items;
    }
    if (lane == 0) dev::tma_store_wait_read();   // no store still reads this CTA's shared memory
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
constexpr int BNW = 128;   // output channels per MMA (its M); a full tile has two such blocks
constexpr int BMX = 256;   // activation rows per tile (MMA N)
constexpr int BK = 64;     // k per TMA stage
constexpr int BKS = 32;    // k per converted sub-block
constexpr int kXStages = 3;    // activation ring, held until the MMAs that read a stage retire
constexpr int kWStages = 4;    // raw-weight ring, held only until a stage is in the converters' registers
constexpr int kCvtBufs = 4;    // converted sub-blocks between the converter warps and the MMA
constexpr int kCvtWarps = 8;    // converter warps per group
constexpr int kCvtGroups = 3;   // group g converts the stages with cnt % 3 == g
constexpr int kCvtSlots = 2;    // converted stages in flight (two sub-block buffers each)
// Warp roles: 0 TMA (activations), 1 MMA issue for channel block 0, 2-25 workers (convert the
// stages of a tile, then drain its accumulators), 26 TMA (raw weights), 27 MMA issue for channel
// block 1.  One thread needs ~85 cycles to issue a tcgen05.mma and about as much per wait and per
// commit, about what the MMAs themselves take; two issuing threads (one per accumulator) leave the
// tensor pipe as the limit.
constexpr int kFirstCvtWarp = 2;
constexpr int kWorkerWarps = kCvtGroups * kCvtWarps;
constexpr int kWProducerWarp = kFirstCvtWarp + kWorkerWarps;
constexpr int kSecondMmaWarp = kWProducerWarp + 1;
constexpr int kWarps = kSecondMmaWarp + 1;
constexpr int kRawBlock = BK * BNW;               // 8 KB  int8 [k][128 n]
constexpr int kRawBytes = 2 * kRawBlock;          // 16 KB: both channel blocks
constexpr int kXBytes = BMX * BK * 2;             // 32 KB bf16 [m][k]
constexpr int kCvtBlock = BKS * BNW * 2;          // 8 KB bf16: two 64-channel halves of [32 k][128 B]
constexpr int kCvtBytes = 2 * kCvtBlock;          // 16 KB: both channel blocks
constexpr int kRawBase = kXStages * kXBytes;                 // 96 KB
constexpr int kCvtBase = kRawBase + kWStages * kRawBytes;    // 160 KB
constexpr int kBarBase = kCvtBase + kCvtBufs * kCvtBytes;    // 224 KB
constexpr int kThreads = kWarps * 32;
constexpr int kSmemBytes = kBarBase + 256 + 1024;
constexpr int kPanelTiles = 8;  // most activation tiles swept together (fewer when K is long: a panel should stay in L2)
// One "consumed" barrier per stage in a ring of 6 (a multiple of both the activation ring and the
// two converted stage slots): the activation producer waits for stage cnt - 3, the converters for
// stage cnt - 2, and the issuing threads commit once per stage.
constexpr int kConsumed = 6;


// Eight int8 (one 8-byte read) -> eight bf16, exactly, in 16 instructions.
// For a byte b (two's complement v): A = 0x4300 | (b & 0x7F) is the bf16
// 128 + (b & 0x7F); C = 0xC300 | (b & 0x80) is -128 for v >= 0 and -256 for
// v < 0; A + C = v, exact in bf16 (|v| <= 128 has 8 significant bits).  One
// byte-permute spreads two bytes over the two halves of a register, two
// logic ops build A and C for both, one packed add finishes the pair.  The MMA
// needs both operands in one 16-bit format (an f16 weight operand against bf16
// activations raises an illegal-instruction error on sm_100a), so the weights
// follow the activations.
__device__ __forceinline__ uint32_t convert2(uint32_t word, uint32_t selector) {
  const uint32_t t = __byte_perm(word, 0u, selector);  // 0x00bb00aa
  uint32_t a, c, r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(a) : "r"(t), "r"(0x007F007Fu), "r"(0x43004300u));  // (t & m) | k
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(c) : "r"(t), "r"(0x00800080u), "r"(0xC300C300u));
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(c));
  return r;
}
__device__ __forceinline__ uint4 convert8(const uint2& in) {
  return make_uint4(convert2(in.x, 0x4140), convert2(in.x, 0x4342), convert2(in.y, 0x4140), convert2(in.y, 0x4342));
}

// The work of one launch.  A full tile is 256 channels x 256 rows: two channel
// blocks share one activation tile, so a CTA stages 48 KB per 64 k for
// 2 x 128 x 256 outputs.  CTA c takes tiles c, c + G, ... for `full_waves`
// rounds; the tiles left over (fewer than G) are cut into `tail_div` parts each
// (1: whole, 2: one channel block, 4: one channel block x 128 rows) and dealt
// round-robin, so that the last round costs 1 / tail_div of a tile.
struct Sched {
  int tiles_n2, tiles_m, full_waves, tail_tiles, tail_div;
  int panel;  // activation tiles per panel
};
struct Work {
  int tn2, tm;   // tile coordinates (256-channel, 256-row units)
  int h0, nh;    // channel blocks [h0, h0 + nh); nh == 0: nothing to do
  int m_off, m_cols;  // rows [m_off, m_off + m_cols) of the activation tile
};

// Tile order: activation tiles are swept in panels of `panel` tiles; inside a
// panel the weight tile changes slowest, so the CTAs that run together share
// one panel of activations (it stays in L2) and a handful of weight tiles.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int panel, int& tm, int& tn) {
  const int per_panel = panel * tiles_n;
  const int p = tile / per_panel, r = tile - p * per_panel;
  const int rows = min(panel, tiles_m - p * panel);  // the last panel may be short
  tn = r / rows;
  tm = p * panel + r % rows;
}

// Item `i` of this CTA; false when the CTA is done.  After its full-wave tiles a CTA takes a
// contiguous run of the tail's parts (tile-major: part 2h + mh of a tile cut in four is channel
// block h, row half mh) and works it off in the largest aligned pieces: a whole tile, a channel
// block with all its rows, or a single part, so that neighbouring parts cost one pipeline fill
// and use the full-width MMA.
__device__ __forceinline__ bool get_work(const Sched& sc, int i, int M, int N, Work& w) {
  const int G = gridDim.x;
  int tile, sub = 0, len = 0;  // len: parts covered, in units of 1 / tail_div tile; 0 = whole tile
  const int div = sc.tail_div;
  if (i < sc.full_waves) {
    tile = blockIdx.x + i * G;
  } else {
    const long long total = static_cast<long long>(sc.tail_tiles) * div;
    int pos = static_cast<int>(blockIdx.x * total / G);
    const int end = static_cast<int>((blockIdx.x + 1) * total / G);
    for (int skip = i - sc.full_waves;; --skip) {
      if (pos >= end) return false;
      const int r = pos % div;
      if (r == 0 && pos + div <= end) len = div;                       // whole tile
      else if (div == 4 && (r & 1) == 0 && pos + 2 <= end) len = 2;    // one channel block, all rows
      else len = 1;
      if (skip == 0) break;
      pos += len;
    }
    tile = sc.full_waves * G + pos / div;
    sub = pos % div;
    if (len == div) len = 0;
  }
  tile_coords(tile, sc.tiles_m, sc.tiles_n2, sc.panel, w.tm, w.tn2);
  w.h0 = 0; w.nh = 2; w.m_off = 0; w.m_cols = BMX;
  if (len != 0) {
    if (div == 2) { w.h0 = sub; w.nh = 1; }
    if (div == 4) {
      w.h0 = sub >> 1; w.nh = 1;
      if (len == 1) { w.m_off = (sub & 1) * (BMX / 2); w.m_cols = BMX / 2; }
    }
  }
  const int blocks_left = (N - w.tn2 * 2 * BNW + BNW - 1) / BNW - w.h0;  // channel blocks that exist
  w.nh = max(0, min(w.nh, blocks_left));
  if (w.tm * BMX + w.m_off >= M) w.nh = 0;
  return true;
}

// Per-group constants of the int4 variant (null / unused for int8 weights).
struct GroupQuant {
  const uint16_t* scales;  // bf16 [K/128, N]
  const uint8_t* zeros;    // u8 [K/128, N], or two per byte [K/128, N/2]
  int packed;
};

// Four packed weights (the two k of two neighbouring channels, one byte per channel, low nibble =
// even k) -> the bf16 pairs (q - z) * s of the even and of the odd k.  0x4300 | q is the bf16
// 128 + q exactly, zz holds 128 + z, so the subtraction is exact and the product is rounded to
// bf16 once: bit for bit what the StableHLO chain convert -> subtract -> multiply computes in bf16.
__device__ __forceinline__ void dequant4(uint32_t t, uint32_t zz, uint32_t ss, uint32_t& even_k, uint32_t& odd_k) {
  uint32_t lo, hi;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(lo) : "r"(t), "r"(0x000F000Fu), "r"(0x43004300u));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(hi) : "r"(t >> 4), "r"(0x000F000Fu), "r"(0x43004300u));
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(lo), "r"(zz));
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(hi), "r"(zz));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(even_k) : "r"(lo), "r"(ss));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(odd_k) : "r"(hi), "r"(ss));
}

// WBITS = 8: int8 weights [K, N], per-channel f32 scale applied in the epilogue.
// WBITS = 4: packed int4 weights [K/2, N] (byte = two k of one channel), per-(128-k group, channel)
//            bf16 scale and zero point applied by the converter warps; K % 128 == 0.
template <int WBITS>
__global__ void __launch_bounds__(kThreads, 1)
w8a16_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
             const float* __restrict__ scale, const GroupQuant gq, uint16_t* __restrict__ y, int M, int N, int K,
             long long ldy, uint32_t idesc256, uint32_t idesc128, const Sched sc, uint32_t flags,
             uint32_t* signal, uint32_t* arrive, int* status) {
  // a raw stage holds 64 k of both channel blocks: 64 byte-rows of int8, 32 of packed int4
  constexpr int kRawRows = (WBITS == 8) ? BK : BK / 2;
  constexpr int kRawBlockW = kRawRows * BNW;
  extern __shared__ uint8_t smem_raw[];
  // An independent launch lets its successor start at once.  A dependent one does so only after
  // its own wait below: a successor that is itself flagged independent can then overlap this
  // launch, but never anything older than it.
  if (flags & QMM_GEMM_INDEPENDENT) dev::pdl_launch_dependents();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* xfull = reinterpret_cast<uint64_t*>(smem + kBarBase);  // activations landed
  uint64_t* wfull = xfull + kXStages;    // raw weights landed
  uint64_t* wempty = wfull + kWStages;   // raw weights are in the converters' registers
  uint64_t* sfull = wempty + kWStages;   // stage ready for the MMAs: converted, and its activations landed
  uint64_t* consumed = sfull + kCvtSlots;   // the MMAs of a stage retired (ring of kConsumed stages)
  uint64_t* tfull = consumed + kConsumed;   // accumulators complete
  uint64_t* tempty = tfull + 1;             // accumulators drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kXStages; ++s) dev::mbar_init(&xfull[s], 1);
    for (int s = 0; s < kWStages; ++s) {
      dev::mbar_init(&wfull[s], 1);
      dev::mbar_init(&wempty[s], kCvtWarps);
    }
    for (int g = 0; g < kCvtSlots; ++g) dev::mbar_init(&sfull[g], kCvtWarps);
    for (int i = 0; i < kConsumed; ++i) dev::mbar_init(&consumed[i], 2);  // one commit per issuing thread
    dev::mbar_init(tfull, 2);
    dev::mbar_init(tempty, kWorkerWarps);
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
  // Ordered behind the kernels ahead on the stream before global memory is touched, unless the
  // caller stated that none of them writes this launch's operands or touches its output.
  if (!(flags & QMM_GEMM_INDEPENDENT)) {
    dev::pdl_wait();
    dev::pdl_launch_dependents();
  }
  const bool mc_store = (flags & QMM_GEMM_STORE_MULTIMEM) != 0;

  // Stage `cnt` (counted over the whole launch) uses activation slot cnt % 3,
  // raw-weight slot cnt % 4 and converted buffers 2 (cnt % 2) and 2 (cnt % 2) + 1.
  if (warp == 0) {
    // ------------------------ TMA producer: activations --------------------
    if (lane == 0) {
      dev::tma_prefetch_desc(&xmap);
      unsigned cnt = 0;
      bool ok = true;
      Work w;
      for (int i = 0; ok && get_work(sc, i, M, N, w); ++i) {
        if (w.nh == 0) continue;
        for (int kb = 0; kb < kblocks; ++kb, ++cnt) {
          const int xs = cnt % kXStages;
          if (cnt >= kXStages) {  // the slot's previous stage must have been multiplied
            const unsigned prev = cnt - kXStages;
            if (!dev::mbar_wait(&consumed[prev % kConsumed], (prev / kConsumed) & 1, status, 21)) { ok = false; break; }
          }
          dev::mbar_expect_tx(&xfull[xs], kXBytes);
          dev::tma_load_2d(smem + xs * kXBytes, &xmap, &xfull[xs], kb * BK, w.tm * BMX);
        }
      }
    }
  } else if (warp == kWProducerWarp) {
    // ------------------------ TMA producer: raw weights --------------------
    if (lane == 0) {
      dev::tma_prefetch_desc(&wmap);
      unsigned cnt = 0;
      bool ok = true;
      Work w;
      for (int i = 0; ok && get_work(sc, i, M, N, w); ++i) {
        if (w.nh == 0) continue;
        for (int kb = 0; kb < kblocks; ++kb, ++cnt) {
          const int ws = cnt & (kWStages - 1);
          if (!dev::mbar_wait(&wempty[ws], ((cnt / kWStages) & 1) ^ 1, status, 20)) { ok = false; break; }
          uint8_t* raw = smem + kRawBase + ws * kRawBytes;
          dev::mbar_expect_tx(&wfull[ws], w.nh * kRawBlockW);
          for (int h = w.h0; h < w.h0 + w.nh; ++h)
            dev::tma_load_2d(raw + h * kRawBlockW, &wmap, &wfull[ws], (w.tn2 * 2 + h) * BNW, kb * kRawRows);
        }
      }
    }
  } else if (warp == 1 || warp == kSecondMmaWarp) {
    // ------------------------------ MMA issuers ----------------------------
    // Issuer j multiplies channel block j of every item that has it into accumulator j; both
    // follow the same barriers and both commit, whether or not they issued anything.  The
    // issuing thread is a slow scalar processor (a branch or a shared-memory poll costs it
    // tens of cycles, a commit ~90), so a stage costs it one wait, one fence, four predicated
    // MMAs with descriptors advanced by adds, and one commit.
    if (lane == 0) {
      const int me = (warp == 1) ? 0 : 1;
      // descriptor halves: the high half is constant, the low half carries the start address
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (kSwizzle128 << 29);  // SBO, version, swizzle
      constexpr uint32_t kAStepK = (16 * 128) >> 4, kAStepH = kCvtBlock >> 4, kAStepBuf = kCvtBytes >> 4;
      constexpr uint32_t kBStepK = 32 >> 4, kBStepStage = kXBytes >> 4;
      const uint32_t a_lo0 = (((dev::smem_u32(smem + kCvtBase) >> 4) & 0x3FFF) | (((BKS * 128u) >> 4) << 16)) +
                             me * kAStepH;
      const uint32_t b_lo0 = ((dev::smem_u32(smem) >> 4) & 0x3FFF) | ((16u >> 4) << 16);
      const uint32_t d = tmem_base + me * BMX;
      uint32_t g = 0, gpar = 0;   // converted-stage slot and the parity of its use
      uint32_t xs = 0;            // activation slot
      uint32_t c6 = 0;            // consumed-ring index
      int items = 0;
      bool ok = true;
      Work w;
      for (int i = 0; ok && get_work(sc, i, M, N, w); ++i) {
        if (w.nh == 0) continue;
        if (!dev::mbar_wait(tempty, (items & 1) ^ 1, status, 22)) break;
        dev::tc_fence_after();
        const uint32_t idesc = (w.m_cols == BMX) ? idesc256 : idesc128;
        const uint32_t b_item = b_lo0 + ((w.m_off * 128) >> 4);
        const uint32_t mine = (me >= w.h0) && (me < w.h0 + w.nh);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!dev::mbar_wait(&sfull[g], gpar, status, 23)) { ok = false; break; }
          dev::tc_fence_after();
          const uint32_t a_c = a_lo0 + g * (2 * kAStepBuf);
          const uint32_t b_s = b_item + xs * kBStepStage;
          dev::umma_f16_lh_if(mine, d, a_c, kDescHi, b_s, kDescHi, idesc, kb != 0);
          dev::umma_f16_lh_if(mine, d, a_c + kAStepK, kDescHi, b_s + kBStepK, kDescHi, idesc, 1);
          dev::umma_f16_lh_if(mine, d, a_c + kAStepBuf, kDescHi, b_s + 2 * kBStepK, kDescHi, idesc, 1);
          dev::umma_f16_lh_if(mine, d, a_c + kAStepBuf + kAStepK, kDescHi, b_s + 3 * kBStepK, kDescHi, idesc, 1);
          dev::tc_commit(&consumed[c6]);  // second arrival: the other issuer
          gpar ^= g;  // the parity flips after slot 1's stage
          g ^= 1;
          xs = (xs == kXStages - 1) ? 0 : xs + 1;
          c6 = (c6 == kConsumed - 1) ? 0 : c6 + 1;
        }
        if (ok) dev::tc_commit(tfull);
        ++items;
      }
    }
  } else {
    // ------------------------------ workers --------------------------------
    // Conversion: a half-warp reads one 128-byte raw row, 8 bytes per lane (conflict-free in any
    // permutation); each lane writes the 16-byte bf16 chunk it made, so a quarter-warp store
    // covers the eight chunks of one 128-byte row of one 64-channel half: conflict-free as well,
    // with no divergence.  One warp needs ~1000 cycles for its share of a stage (dependent ALU
    // chains), as long as the MMAs of the stage take, so three groups of eight warps take every
    // third stage.  The raw slot is handed back as soon as its bytes are in registers.
    // Epilogue: when the tile's stages are converted the same 24 warps drain its accumulators
    // (warp & 3 selects the 32 TMEM lanes = channels a warp may read; the six warps of a lane
    // quarter share the 32-row chunks).
    const int o = warp - kFirstCvtWarp;
    const int grp = o / kCvtWarps, cw = o % kCvtWarps;
    const int q = warp & 3, esub = o >> 2;
    const int piece = lane & 15;         // 8 channels: [8*piece, 8*piece+8)
    const int rsub = lane >> 4;          // row within a pair
    unsigned cnt = 0;  // stages since the start of the launch
    int r3 = 0;        // cnt % 3
    int items = 0;
    bool ok = true;
    Work w;
    for (int i = 0; ok && get_work(sc, i, M, N, w); ++i) {
      if (w.nh == 0) continue;
      for (int kb = 0; kb < kblocks; ++kb, ++cnt, r3 = (r3 == 2) ? 0 : r3 + 1) {
        if (r3 != grp) continue;
        const int ws = cnt & (kWStages - 1);
        const int slot = cnt & 1, c0 = 2 * slot;  // the stage's two converted buffers
        const uint8_t* raw = smem + kRawBase + ws * kRawBytes;
        if constexpr (WBITS == 4) {
          // ---- packed int4: a lane owns 8 channels of each channel block; a byte-row of the raw
          // tile (two k per byte) becomes two k-rows of the converted tile.  Scales and zero points
          // of the stage's 128-k group are fetched before the wait for the weights.
          const int grp_q = kb >> 1;
          uint4 sv[2];
          uint2 zv[2];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            sv[hh] = make_uint4(0, 0, 0, 0);
            zv[hh] = make_uint2(0, 0);
            if (hh < w.nh) {
              const long long n0 = static_cast<long long>(w.tn2 * 2 + w.h0 + hh) * BNW + piece * 8;
              sv[hh] = __ldg(reinterpret_cast<const uint4*>(gq.scales + static_cast<long long>(grp_q) * N + n0));
              if (gq.packed) zv[hh].x = __ldg(reinterpret_cast<const uint32_t*>(gq.zeros + (static_cast<long long>(grp_q) * N + n0) / 2));
              else zv[hh] = __ldg(reinterpret_cast<const uint2*>(gq.zeros + static_cast<long long>(grp_q) * N + n0));
            }
          }
          if (!dev::mbar_wait_warp(&wfull[ws], (cnt / kWStages) & 1, status, 26)) { ok = false; break; }
          uint2 in[4];  // [sub-block][channel block]
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int sb = p >> 1, hh = p & 1;
            const int brow = sb * (BKS / 2) + cw * 2 + rsub;  // byte-row 0..31 of the stage
            in[p] = make_uint2(0, 0);
            if (hh < w.nh)
              in[p] = *reinterpret_cast<const uint2*>(raw + (w.h0 + hh) * kRawBlockW + brow * 128 +
                                                      (((piece >> 1) ^ (brow & 7)) << 4) + ((piece & 1) << 3));
          }
          __syncwarp();
          if (lane == 0) dev::mbar_arrive(&wempty[ws]);  // every raw byte of the stage is in registers
          bool waited = false;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            if (hh >= w.nh) continue;
            // 128 + z and s of the lane's four channel pairs
            uint32_t zz[4], ss[4] = {sv[hh].x, sv[hh].y, sv[hh].z, sv[hh].w};
            if (gq.packed) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t b = (zv[hh].x >> (8 * j)) & 0xFFu;  // channels 2j (low nibble), 2j+1 (high)
                zz[j] = 0x43004300u | (b & 0xFu) | ((b >> 4) << 16);
              }
            } else {
              zz[0] = __byte_perm(zv[hh].x, 0x43004300u, 0x7150);
              zz[1] = __byte_perm(zv[hh].x, 0x43004300u, 0x7352);
              zz[2] = __byte_perm(zv[hh].y, 0x43004300u, 0x7150);
              zz[3] = __byte_perm(zv[hh].y, 0x43004300u, 0x7352);
            }
#pragma unroll
            for (int sb = 0; sb < 2; ++sb) {
              const uint2 v = in[sb * 2 + hh];
              uint4 ev, od;
              dequant4(__byte_perm(v.x, 0u, 0x4140), zz[0], ss[0], ev.x, od.x);
              dequant4(__byte_perm(v.x, 0u, 0x4342), zz[1], ss[1], ev.y, od.y);
              dequant4(__byte_perm(v.y, 0u, 0x4140), zz[2], ss[2], ev.z, od.z);
              dequant4(__byte_perm(v.y, 0u, 0x4342), zz[3], ss[3], ev.w, od.w);
              if (!waited) {
                waited = true;
                if (cnt >= 2) {  // the MMAs of the stage that used these buffers before must have retired
                  const unsigned prev = cnt - 2;
                  if (!dev::mbar_wait_warp(&consumed[prev % kConsumed], (prev / kConsumed) & 1, status, 27)) ok = false;
                }
              }
              if (ok) {
                uint8_t* cvt = smem + kCvtBase + (c0 + sb) * kCvtBytes + (w.h0 + hh) * kCvtBlock +
                               (piece >> 3) * (BKS * 128);
                const int r = 2 * (cw * 2 + rsub);  // k-row of the even k inside the 32-k sub-block
                *reinterpret_cast<uint4*>(cvt + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) = ev;
                *reinterpret_cast<uint4*>(cvt + (r + 1) * 128 + (((piece & 7) ^ ((r + 1) & 7)) << 4)) = od;
              }
            }
          }
          if (!ok) break;
        } else {
        if (!dev::mbar_wait_warp(&wfull[ws], (cnt / kWStages) & 1, status, 26)) { ok = false; break; }
        // tasks of this warp: per sub-block and channel block 16 row pairs, two per warp
        uint2 in[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const int sb = p >> 2, hh = (p >> 1) & 1;  // sub-block; 0: first block of the item, 1: second
          const int r = ((p & 1) * kCvtWarps + cw) * 2 + rsub;  // row 0..31 of the sub-block
          const int krow = sb * BKS + r;
          if (hh < w.nh)
            in[p] = *reinterpret_cast<const uint2*>(raw + (w.h0 + hh) * kRawBlockW + krow * 128 +
                                                    (((piece >> 1) ^ (krow & 7)) << 4) + ((piece & 1) << 3));
        }
        // sub-block 0 is converted before the wait for its buffers, sub-block 1 after its stores
        uint4 out[4];
#pragma unroll
        for (int p = 0; p < 4; ++p)
          if ((p >> 1) < w.nh) out[p] = convert8(in[p]);
        if (cnt >= 2) {  // the MMAs of the stage that used these buffers before must have retired
          const unsigned prev = cnt - 2;
          if (!dev::mbar_wait_warp(&consumed[prev % kConsumed], (prev / kConsumed) & 1, status, 27)) { ok = false; break; }
        }
#pragma unroll
        for (int sb = 0; sb < 2; ++sb) {
          uint8_t* cvt = smem + kCvtBase + (c0 + sb) * kCvtBytes;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int hh = p >> 1;
            const int r = ((p & 1) * kCvtWarps + cw) * 2 + rsub;
            if (hh < w.nh)
              *reinterpret_cast<uint4*>(cvt + (w.h0 + hh) * kCvtBlock + (piece >> 3) * (BKS * 128) + r * 128 +
                                        (((piece & 7) ^ (r & 7)) << 4)) = out[p];
          }
          if (sb == 0) {
#pragma unroll
            for (int p = 0; p < 4; ++p)
              if ((p >> 1) < w.nh) out[p] = convert8(in[4 + p]);
            // every raw byte of the stage is in registers: hand the slot back
            __syncwarp();
            if (lane == 0) dev::mbar_arrive(&wempty[ws]);
          }
        }
        }
        dev::fence_proxy_async();
        // the issuing threads wait only for this barrier: make sure the activations are there too
        if (!dev::mbar_wait_warp(&xfull[cnt % kXStages], (cnt / kXStages) & 1, status, 28)) { ok = false; break; }
        __syncwarp();
        if (lane == 0) dev::mbar_arrive(&sfull[slot]);
      }
      if (!ok) break;
      // ---- epilogue of this item
      if (!dev::mbar_wait_relaxed_warp(tfull, items & 1, status, 25)) break;
      dev::tc_fence_after();
      const int chunks = w.m_cols / 32;
#pragma unroll 1
      for (int idx = esub; idx < w.nh * chunks; idx += kWorkerWarps / 4) {
        const int h = w.h0 + idx / chunks, ch = idx % chunks;
        const int n = (w.tn2 * 2 + h) * BNW + q * 32 + lane;  // this thread's output channel
        const float scl = (WBITS == 4) ? 1.f : ((n < N) ? __ldg(scale + n) : 0.f);
        uint32_t r[32];
        dev::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * BMX + ch * 32, r);
        dev::tc_wait_ld();
        const int m0 = w.tm * BMX + w.m_off + ch * 32;
        // pair neighbouring channels so that every lane stores 4 bytes: even
        // lanes write rows m0+2j, odd lanes rows m0+2j+1
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a = __uint_as_float(r[2 * j]) * scl;
          const float b = __uint_as_float(r[2 * j + 1]) * scl;
          const float send = (lane & 1) ? a : b;
          const float got = __shfl_xor_sync(0xFFFFFFFFu, send, 1);
          const int m = m0 + 2 * j + (lane & 1);
          const uint32_t packed = (lane & 1) ? dev::pack_bf16x2(got, b) : dev::pack_bf16x2(a, got);
          const int n_even = n & ~1;
          if (m < M && n_even < N) {
            uint16_t* dst = y + static_cast<size_t>(m) * ldy + n_even;
            if (mc_store) dev::multimem_st_b32(dst, packed);  // the same offset of every rank's buffer
            else *reinterpret_cast<uint32_t*>(dst) = packed;
          }
        }
      }
      dev::tc_fence_before();
      __syncwarp();
      if (lane == 0) dev::mbar_arrive(tempty);
      ++items;
    }
  }
  // Completion signal: every thread that stored makes its stores visible system-wide, the CTAs
  // count themselves on a local counter (which wraps back to zero), and the last one adds 1 to
  // the signal word with release semantics: on every rank at once when the word is a multicast
  // address.  A reader that sees the new count with an acquire load sees the whole output block.
  if (signal != nullptr) dev::fence_sys();
  dev::tc_fence_before();
  __syncthreads();
  if (warp == 1) dev::tmem_dealloc(tmem_base, 512);
  if (signal != nullptr && threadIdx.x == 0) {
    const unsigned prev = atomicInc(arrive, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      dev::fence_sys();
      if (mc_store) dev::multimem_red_release_add_u32(signal, 1u);
      else dev::red_release_sys_add_u32(signal, 1u);
    }
  }
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
                                  (uint64_t)K, (uint64_t)K, BMB, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&bmap, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K,
                                  (uint64_t)N, (uint64_t)N, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // results leave through TMA stores of 32 x 32 chunks (128 bytes of a row per chunk)
  CUtensorMap accmap = amap, outmap = amap;   // placeholders where an output is absent (never used by the kernel)
  if (acc)
    if (int rc = make_tensor_map_2d(&accmap, acc, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, (uint64_t)M, (uint64_t)N,
                                    (uint64_t)N * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  if (out)
    if (int rc = make_tensor_map_2d(&outmap, out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)M, (uint64_t)N,
                                    (uint64_t)N * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  static std::atomic<uint64_t> configured{0};  // per device
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(i8gemm_kernel), kSmemBytes, configured)) return rc;
  const uint32_t idesc = dev::make_idesc(/*c=s32*/ 2, a_unsigned ? 0 : 1, b_unsigned ? 0 : 1,
                                         /*a K-major*/ 0, /*b MN-major*/ 1, BMB, BN);
  const int tiles = static_cast<int>(((M + 2 * BMB - 1) / (2 * BMB)) * ((N + BN - 1) / BN));
  const int ctas = gemm_ctas();
  const int halves = (tiles * 2 <= ctas) ? 1 : 0;  // few tiles: one row block per CTA
  const int items = tiles * (halves ? 2 : 1);
  const int grid = items < ctas ? items : ctas;
  static std::atomic<int> staged_cache{INT32_MIN};
  const int staged = env_int_once("QMM_I8_STAGED_STORE", 1, staged_cache);   // 0: results stored straight from registers
  i8gemm_kernel<<<grid, kThreads, kSmemBytes, stream>>>(amap, bmap, accmap, outmap, acc, out, row_scale, col_scale,
                                                        (int)M, (int)N, (int)K, idesc, halves, staged,
                                                        device_status_word());
  QMM_CHECK_LAUNCH("i8gemm_kernel");
  return QMM_OK;
}

// Shared launch path of the weight-only GEMMs (int8 per-channel, int4 group-wise).
template <int WBITS>
static int launch_weight_only(const uint16_t* x, const void* w, const float* scale, const tc::w8::GroupQuant& gq,
                              uint16_t* y, int64_t M, int64_t N, int64_t K, int64_t ldy, uint32_t flags,
                              uint32_t* signal, uint32_t* arrive, cudaStream_t stream) {
  using namespace tc::w8;
  CUtensorMap wmap, xmap;
  constexpr int kRawRows = (WBITS == 8) ? BK : BK / 2;
  if (int rc = make_tensor_map_2d(&wmap, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)(WBITS == 8 ? K : K / 2),
                                  (uint64_t)N, (uint64_t)N, kRawRows, BNW, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map_2d(&xmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M,
                                  (uint64_t)K, (uint64_t)K * 2, BMX, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  static std::atomic<uint64_t> configured{0};  // per device (one mask per template instance)
  auto kern = w8a16_kernel<WBITS>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kSmemBytes, configured)) return rc;
  // operand "a" of the MMA = weights (bf16, MN-major), "b" = activations (bf16, K-major)
  const uint32_t idesc256 = dev::make_idesc(/*c=f32*/ 1, /*bf16*/ 1, /*bf16*/ 1,
                                            /*a MN-major*/ 1, /*b K-major*/ 0, BNW, BMX);
  const uint32_t idesc128 = dev::make_idesc(1, 1, 1, 1, 0, BNW, BMX / 2);
  Sched sc;
  sc.tiles_n2 = static_cast<int>((N + 2 * BNW - 1) / (2 * BNW));
  sc.tiles_m = static_cast<int>((M + BMX - 1) / BMX);
  const int tiles = sc.tiles_n2 * sc.tiles_m;
  {
    // a panel of activation tiles (256 rows x K bf16 each) should fit in half of L2 (measured at
    // K = 28672, N = 8192: panels of 8 / 4 / 3 / 2 tiles give 1180 / 1218 / 1149 / 1134 TFLOP/s)
    const long long tile_bytes = 2ll * BMX * K;
    long long pt = (64ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
    sc.panel = static_cast<int>(pt < 2 ? 2 : (pt > kPanelTiles ? kPanelTiles : pt));
  }
  const int sms = gemm_ctas();  // persistent CTAs of this launch
  sc.full_waves = tiles / sms;
  sc.tail_tiles = tiles - sc.full_waves * sms;
  // cut the leftover tiles as finely as shortens the last round
  sc.tail_div = 1;
  int best_num = 1, best_den = 1;  // cost of the last round = rounds / parts, in tiles
  for (int d = 2; d <= 4 && sc.tail_tiles > 0; d *= 2) {
    const int rounds = (sc.tail_tiles * d + sms - 1) / sms;
    if (rounds * best_den < best_num * d) {
      best_num = rounds;
      best_den = d;
      sc.tail_div = d;
    }
  }
  const int grid = sc.full_waves > 0 ? sms : (sc.tail_tiles * sc.tail_div < sms ? sc.tail_tiles * sc.tail_div : sms);
  // Programmatic stream serialization: the CTAs of this launch may become resident while the
  // kernel ahead of it drains; they order themselves behind it inside the kernel (or not at all
  // when the caller states independence, which fills the last, partly idle round of one launch
  // with the first tiles of the next).
  QMM_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(kThreads), kSmemBytes, stream, wmap, xmap, scale, gq, y, (int)M,
                          (int)N, (int)K, (long long)ldy, idesc256, idesc128, sc, flags, signal, arrive,
                          device_status_word()));
  return QMM_OK;
}

int w8a16_tcgen05(const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y, int64_t M,
                  int64_t N, int64_t K, int64_t ldy, uint32_t flags, uint32_t* signal, uint32_t* arrive,
                  cudaStream_t stream) {
  const tc::w8::GroupQuant none = {nullptr, nullptr, 0};
  return launch_weight_only<8>(x, w, scale, none, y, M, N, K, ldy, flags, signal, arrive, stream);
}

// int4 g128 weight-only GEMM for prefill-sized M: same pipeline, nibbles dequantised by the
// converter warps.  Requires K % 128 == 0 and N % 128 == 0 (checked by the caller).
int w4a16_tcgen05(const uint16_t* x, const uint8_t* wq, const uint16_t* scales, const uint8_t* zeros,
                  int zeros_packed, uint16_t* y, int64_t M, int64_t N, int64_t K, uint32_t flags,
                  cudaStream_t stream) {
  const tc::w8::GroupQuant gq = {scales, zeros, zeros_packed};
  return launch_weight_only<4>(x, wq, nullptr, gq, y, M, N, K, N, flags, nullptr, nullptr, stream);
}

}  // namespace qmm
