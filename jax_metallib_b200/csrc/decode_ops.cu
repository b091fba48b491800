// The non-matmul operators of a Llama-shaped decode step (bf16 activations):
// embedding row gather, (residual add +) RMSNorm, rotary embedding, SwiGLU
// gating, grouped-query decode attention over a read-only KV cache, and a
// bf16 matmul for a few activation rows (the unquantized lm_head).
// They are small next to the int4 linears; each is one launch, written to be
// captured in a CUDA graph together with the quantized matmuls.  Every kernel
// here is launched with programmatic stream serialization: it lets the next
// kernel start at once (so that a following int4 matmul streams its weights
// while this one runs) and waits for its predecessors before touching data.
//
// Reference semantics kept where the reference pins them: take-rows wraps
// negative indices and fills out-of-range rows
// (README.md:200-202, core/mps_executable.mm:1149-1160); the new K/V rows are
// returned separately and the cache is a read-only input, because the
// reference has no buffer donation (api/pjrt_api.cc:310) and a
// dynamic_update_slice of the whole cache per token would copy 2 GB.
#include <math.h>

#include "common.cuh"

namespace qmm {
namespace dec {

__device__ __forceinline__ float2 bf2_to_f2(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}

// ---------------------------------------------------------------------------
// take rows: out[b, :] = table[wrap(ids[b]), :] or fill
// ---------------------------------------------------------------------------
__global__ void take_rows_kernel(const uint16_t* __restrict__ table, const int32_t* __restrict__ ids,
                                 uint16_t* __restrict__ out, int V, int D, uint16_t fill_bits) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  const int b = blockIdx.x;
  int id = ids[b];
  if (id < 0) id += V;  // negative indices count from the end
  const bool valid = id >= 0 && id < V;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(valid ? id : 0) * D);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(b) * D);
  const uint32_t f2 = fill_bits | (static_cast<uint32_t>(fill_bits) << 16);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = valid ? __ldg(src + i) : make_uint4(f2, f2, f2, f2);
}

// ---------------------------------------------------------------------------
// h = x (+ r);  y = bf16( float(bf16(h * rsqrt(mean(h^2) + eps))) * w )
// ---------------------------------------------------------------------------
constexpr int kNormThreads = 1024, kNormPairs = 8;  // a row of up to 16384 values lives in registers

__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ r,
                   const uint16_t* __restrict__ w, uint16_t* __restrict__ sum_out,
                   uint16_t* __restrict__ norm_out, int D, float eps) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  const int row = blockIdx.x;
  const uint32_t* xp = reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(row) * D);
  const uint32_t* rp = r ? reinterpret_cast<const uint32_t*>(r + static_cast<size_t>(row) * D) : nullptr;
  const uint32_t* wp = reinterpret_cast<const uint32_t*>(w);
  __shared__ float red[kNormThreads / 32];
  float2 h[kNormPairs];  // the (rounded) sum row, this thread's pairs
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kNormPairs; ++it) {
    const int i = threadIdx.x + it * kNormThreads;
    h[it] = make_float2(0.f, 0.f);
    if (i < D / 2) {
      float2 a = bf2_to_f2(__ldg(xp + i));
      if (rp) {
        const float2 b = bf2_to_f2(__ldg(rp + i));
        // the residual stream is kept in bf16: round the sum once
        const uint32_t s = dev::pack_bf16x2(a.x + b.x, a.y + b.y);
        if (sum_out) reinterpret_cast<uint32_t*>(sum_out + static_cast<size_t>(row) * D)[i] = s;
        a = bf2_to_f2(s);
      }
      h[it] = a;
      ss += a.x * a.x + a.y * a.y;
    }
  }
  for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = (threadIdx.x & 31) < kNormThreads / 32 ? red[threadIdx.x & 31] : 0.f;
  for (int off = 16; off >= 1; off >>= 1) tot += __shfl_xor_sync(0xFFFFFFFFu, tot, off);
  const float inv = rsqrtf(tot / static_cast<float>(D) + eps);
#pragma unroll
  for (int it = 0; it < kNormPairs; ++it) {
    const int i = threadIdx.x + it * kNormThreads;
    if (i < D / 2) {
      const float2 g = bf2_to_f2(__ldg(wp + i));
      const float2 n = bf2_to_f2(dev::pack_bf16x2(h[it].x * inv, h[it].y * inv));
      reinterpret_cast<uint32_t*>(norm_out + static_cast<size_t>(row) * D)[i] = dev::pack_bf16x2(n.x * g.x, n.y * g.y);
    }
  }
}

// ---------------------------------------------------------------------------
// rotary embedding, rotate-half pairing (i, i + hd/2), in place on q and k;
// one thread per (batch row, head, pair); q / k batch rows are q_ld / k_ld
// elements apart (they may be slices of one fused projection output)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(uint16_t* __restrict__ q, uint16_t* __restrict__ k, const int32_t* __restrict__ pos, int B, int Hq,
            int Hkv, int hd, float theta, long long q_ld, long long k_ld) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  const int half = hd / 2;
  const int per_row = (Hq + Hkv) * half;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * per_row) return;
  const int b = idx / per_row, i = idx % per_row;
  const int h = i / half, j = i % half;
  uint16_t* base = (h < Hq) ? q + static_cast<size_t>(b) * q_ld + static_cast<size_t>(h) * hd
                            : k + static_cast<size_t>(b) * k_ld + static_cast<size_t>(h - Hq) * hd;
  const float p = static_cast<float>(pos[b]);
  const float freq = powf(theta, -2.0f * static_cast<float>(j) / static_cast<float>(hd));
  float sn, cs;
  sincosf(p * freq, &sn, &cs);
  const float a = dev::bf16_bits_to_float(base[j]), c = dev::bf16_bits_to_float(base[j + half]);
  base[j] = dev::float_to_bf16_bits(a * cs - c * sn);
  base[j + half] = dev::float_to_bf16_bits(c * cs + a * sn);
}

// ---------------------------------------------------------------------------
// out = bf16( silu(gate) * up ), silu(x) = x * sigmoid(x); gate/up may be the
// two halves of one [B, 2F] buffer (ld = row stride in elements)
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                                uint16_t* __restrict__ out, int F, long long ld_in) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= F / 2) return;
  const float2 g = bf2_to_f2(reinterpret_cast<const uint32_t*>(gate + static_cast<size_t>(row) * ld_in)[i]);
  const float2 u = bf2_to_f2(reinterpret_cast<const uint32_t*>(up + static_cast<size_t>(row) * ld_in)[i]);
  // the activation is rounded to bf16 before the product, as an un-fused bf16 graph does
  const float2 s = bf2_to_f2(dev::pack_bf16x2(g.x / (1.f + __expf(-g.x)), g.y / (1.f + __expf(-g.y))));
  reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row) * F)[i] = dev::pack_bf16x2(s.x * u.x, s.y * u.y);
}

// ---------------------------------------------------------------------------
// decode attention, grouped-query, head dim 128.
//   cache k/v: [B, Hkv, L, 128] bf16 (read only); new row knew/vnew [B, Hkv, 128]
//   q [B, Hq, 128] -> out [B, Hq, 128]; the new row is the (L+1)-th key.
// Pass 1 (attn_partial): the cache rows of one (b, kv head) are cut into
// `nsplit` contiguous runs of 64-row tiles; one CTA streams a run through a
// three-stage TMA ring (K and V tile, 16 KB each, 128-byte swizzle).  Four
// consumer warps each own 16 rows of every tile and keep their own running
// softmax (max, sum, 128-dim accumulator) for the R = Hq/Hkv query heads that
// share the kv head, on the tensor cores (mma.sync m16n8k16, bf16):
//   S^T[head, row] = Q[head, d] . K[row, d]     (heads padded to 16, A = Q in registers)
//   O[head, d]    += P[head, row] . V[row, d]   (P straight from the S^T accumulators)
// so the kernel does ~32 MMAs per 8 KB of cache and stays HBM-bound.  The
// warps merge through shared memory and write one (max, sum, O) partial per
// (b, head, split).  Pass 2 (attn_combine) merges the splits and the new row.
// ---------------------------------------------------------------------------
constexpr int kHd = 128, kTileRows = 64, kAttnStages = 3, kAttnWarps = 4;
constexpr int kAttnStageBytes = 2 * kTileRows * kHd * 2;  // K tile + V tile = 32 KB
constexpr int kAttnSmem = kAttnStages * kAttnStageBytes + 128 + 1024;
constexpr int kAttnThreads = (kAttnWarps + 1) * 32;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D += A.B with the lower eight rows of A (a1, a3) zero: only query heads 0..7 exist
__device__ __forceinline__ void mma_heads(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, "
      "{%7, %8}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}

// tiles [begin, end) of split `s` out of `nsplit` over `ntiles`
__host__ __device__ inline int split_begin(int s, int nsplit, int ntiles) {
  return static_cast<int>(static_cast<long long>(s) * ntiles / nsplit);
}

__global__ void __launch_bounds__(kAttnThreads)
attn_partial_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                    const uint16_t* __restrict__ q, float* __restrict__ part, int Hq, int Hkv, int R, int L,
                    int nsplit, float scale, long long q_ld, int static_cache, int* status) {
  dev::pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kAttnStages * kAttnStageBytes);
  uint64_t* empty = full + kAttnStages;

  const int split = blockIdx.x, bh = blockIdx.y;  // bh = b * Hkv + kvh
  const int b = bh / Hkv, kvh = bh % Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (L + kTileRows - 1) / kTileRows;
  const int t_begin = split_begin(split, nsplit, ntiles), t_end = split_begin(split + 1, nsplit, ntiles);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAttnStages; ++s) {
      dev::mbar_init(&full[s], 1);
      dev::mbar_init(&empty[s], kAttnWarps);
    }
    dev::fence_mbar_init();
  }
  __syncthreads();

  if (warp == kAttnWarps) {
    // ------------------------------ producer -------------------------------
    // A cache that no kernel still in flight writes can be fetched before the
    // kernels ahead on the stream have finished.
    if (!static_cache) dev::pdl_wait();
    if (lane == 0) {
      const uint64_t policy = dev::policy_evict_first();
      int s = 0;
      uint32_t ph = 0;
      for (int t = t_begin; t < t_end; ++t) {
        if (!dev::mbar_wait_relaxed(&empty[s], ph ^ 1, status, 31)) break;
        uint8_t* st = smem + s * kAttnStageBytes;
        const int grow = bh * L + t * kTileRows;  // row in the [B*Hkv*L, 128] view
        dev::mbar_expect_tx(&full[s], kAttnStageBytes);
        dev::tma_load_2d_hint(st, &kmap, &full[s], 0, grow, policy);
        dev::tma_load_2d_hint(st + 8192, &kmap, &full[s], 64, grow, policy);
        dev::tma_load_2d_hint(st + 16384, &vmap, &full[s], 0, grow, policy);
        dev::tma_load_2d_hint(st + 24576, &vmap, &full[s], 64, grow, policy);
        if (++s == kAttnStages) { s = 0; ph ^= 1; }
      }
    }
    return;
  }

  // -------------------------------- consumers -------------------------------
  dev::pdl_wait();  // q comes from the kernels ahead; the partials go to a shared workspace
  const int g8 = lane >> 2, t4 = lane & 3;  // this thread's head (if g8 < R) and column pair
  // Q fragments of the A operand: head g8, d = 16 ks + 2 t4 (+1) and + 8
  uint32_t qa[8][2];
  {
    const uint16_t* qrow = q + static_cast<size_t>(b) * q_ld + static_cast<size_t>(kvh * R + g8) * kHd;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = g8 < R ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4) : 0u;
      qa[ks][1] = g8 < R ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4 + 8) : 0u;
    }
  }
  const float sl2 = scale * 1.4426950408889634f;  // scores in log2 units
  float m_run = -INFINITY, l_run = 0.f;
  float o[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nt][i] = 0.f;

  // ldmatrix lane roles
  const int mi = lane >> 3, rin = lane & 7;
  const int krow = warp * 16 + (mi >> 1) * 8 + rin;  // K: matrices (rows lo, d lo), (rows lo, d hi), (rows hi, d lo), (rows hi, d hi)
  const int kchunk = mi & 1;
  const int vrow = warp * 16 + (mi & 1) * 8 + rin;   // V: (rows lo, d), (rows hi, d), (rows lo, d + 8), (rows hi, d + 8)
  const int vchunk = mi >> 1;

  int s = 0;
  uint32_t ph = 0;
  for (int t = t_begin; t < t_end; ++t) {
    if (!dev::mbar_wait_relaxed_warp(&full[s], ph, status, 32)) return;
    const uint32_t kb = dev::smem_u32(smem + s * kAttnStageBytes);
    const uint32_t vb = kb + 16384;
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sacc[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int c16 = 2 * ks + kchunk;  // 16-byte chunk of the 256-byte row
      uint32_t r[4];
      ldsm_x4(kb + (c16 >> 3) * 8192 + krow * 128 + (((c16 & 7) ^ (krow & 7)) << 4), r);
      mma_heads(sacc[0], qa[ks][0], qa[ks][1], r[0], r[1]);
      mma_heads(sacc[1], qa[ks][0], qa[ks][1], r[2], r[3]);
    }
    // sacc[nt][0..1] = scores of head g8 against rows 16 warp + 8 nt + 2 t4 (+1)
    const int row0 = t * kTileRows + warp * 16 + 2 * t4;
    float tv[2][2], tmax = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        tv[nt][i] = (row0 + 8 * nt + i < L) ? sacc[nt][i] * sl2 : -INFINITY;
        tmax = fmaxf(tmax, tv[nt][i]);
      }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 2));
    const float m_new = fmaxf(m_run, tmax);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // a slab with no valid row yet
    const float alpha = exp2f(m_run - m_use);
    float p[2][2], psum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        p[nt][i] = exp2f(tv[nt][i] - m_use);
        psum += p[nt][i];
      }
    psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 1);
    psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      o[nt][0] *= alpha;
      o[nt][1] *= alpha;
    }
    const uint32_t pa0 = dev::pack_bf16x2(p[0][0], p[0][1]);  // rows 2 t4 (+1)
    const uint32_t pa2 = dev::pack_bf16x2(p[1][0], p[1][1]);  // rows 8 + 2 t4 (+1)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c16 = 2 * j + vchunk;
      uint32_t r[4];
      ldsm_x4_t(vb + (c16 >> 3) * 8192 + vrow * 128 + (((c16 & 7) ^ (vrow & 7)) << 4), r);
      mma_heads(o[2 * j], pa0, pa2, r[0], r[1]);
      mma_heads(o[2 * j + 1], pa0, pa2, r[2], r[3]);
    }
    __syncwarp();
    if (lane == 0) dev::mbar_arrive(&empty[s]);
    if (++s == kAttnStages) { s = 0; ph ^= 1; }
  }

  // merge the four warps through the (now idle) first ring stage:
  // mrg[warp][head][2 + 128] = (max, sum, o)
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnWarps * 32));  // every warp is past its last tile read
  float* mrg = reinterpret_cast<float*>(smem);
  if (g8 < R) {
    float* dst = mrg + (warp * R + g8) * (kHd + 2);
    if (t4 == 0) {
      dst[0] = m_run;
      dst[1] = l_run;
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<float2*>(dst + 2 + 8 * nt + 2 * t4) = make_float2(o[nt][0], o[nt][1]);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnWarps * 32));
  // part layout: [bh][split][head][2 + 128] = (max in natural-log units, sum, o[128])
  const int d = threadIdx.x;  // 0..127
  for (int h = 0; h < R; ++h) {
    float mw[kAttnWarps], m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      mw[w] = mrg[(w * R + h) * (kHd + 2)];
      m_tot = fmaxf(m_tot, mw[w]);
    }
    float l_tot = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float wgt = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - m_tot);
      l_tot = fmaf(wgt, mrg[(w * R + h) * (kHd + 2) + 1], l_tot);
      acc = fmaf(wgt, mrg[(w * R + h) * (kHd + 2) + 2 + d], acc);
    }
    float* dst = part + ((static_cast<size_t>(bh) * nsplit + split) * R + h) * (kHd + 2);
    dst[2 + d] = acc;
    if (d == 0) {
      dst[0] = m_tot * 0.6931471805599453f;
      dst[1] = l_tot;
    }
  }
}

// one block per (b, q head): merge the splits and the new key/value row
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* __restrict__ part, const uint16_t* __restrict__ q,
                    const uint16_t* __restrict__ knew, const uint16_t* __restrict__ vnew,
                    uint16_t* __restrict__ out, int Hq, int Hkv, int R, int nsplit, float scale, long long q_ld,
                    long long new_ld) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  const int b = blockIdx.x / Hq, hq = blockIdx.x % Hq;
  const int kvh = hq / R, h = hq % R;
  const int bh = b * Hkv + kvh;
  const int d = threadIdx.x;
  __shared__ float red[4];
  // score of the new row
  const float qd = dev::bf16_bits_to_float(q[static_cast<size_t>(b) * q_ld + static_cast<size_t>(hq) * kHd + d]);
  const float kd = dev::bf16_bits_to_float(knew[static_cast<size_t>(b) * new_ld + static_cast<size_t>(kvh) * kHd + d]);
  float s = qd * kd;
  for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
  if ((d & 31) == 0) red[d >> 5] = s;
  __syncthreads();
  const float s_new = (red[0] + red[1] + red[2] + red[3]) * scale;
  float m = s_new;
  const float* base = part + (static_cast<size_t>(bh) * nsplit * R + h) * (kHd + 2);
  const size_t stride = static_cast<size_t>(R) * (kHd + 2);
  for (int c = 0; c < nsplit; ++c) m = fmaxf(m, base[c * stride]);
  float denom = __expf(s_new - m);
  float acc = denom * dev::bf16_bits_to_float(vnew[static_cast<size_t>(b) * new_ld + static_cast<size_t>(kvh) * kHd + d]);
  for (int c = 0; c < nsplit; ++c) {
    const float* p = base + c * stride;
    const float wgt = __expf(p[0] - m);
    denom = fmaf(wgt, p[1], denom);
    acc = fmaf(wgt, p[2 + d], acc);
  }
  out[(static_cast<size_t>(b) * Hq + hq) * kHd + d] = dev::float_to_bf16_bits(acc / denom);
}

// ---------------------------------------------------------------------------
// y[M,N] = x[M,K] @ w[K,N], bf16 in, f32 accumulate, bf16 out, M <= 16.
// HBM-bound on w (read once).  One CTA owns 128 columns and all of K; a
// producer thread streams 64-k tiles (two 64-column boxes, 128-byte swizzle)
// plus the matching activation tile; four consumer warps own 32 columns each:
// ldmatrix.trans makes the [k][n] tile the 16-row MMA operand, the activations
// are the 8-column operand (mma.sync.m16n8k16).
// ---------------------------------------------------------------------------
namespace gemv {
constexpr int BN = 128, BK = 64, kStages = 5;
constexpr int kWBytes = BK * BN * 2;  // 16 KB: two [64 k][64 n] boxes
constexpr int kXBytes = 16 * BK * 2;  // 2 KB: [16 rows][64 k]
constexpr int kStage = kWBytes + kXBytes;  // 18 KB, a multiple of 1024
constexpr int kSmem = kStages * kStage + 1024 + 1024;

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MT>
__global__ void __launch_bounds__(160)
bf16_small_m_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                    uint16_t* __restrict__ y, int M, int N, int K, int* status) {
  dev::pdl_launch_dependents();
  dev::pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStage);
  uint64_t* empty = full + kStages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int kblocks = K / BK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      dev::mbar_init(&full[s], 1);
      dev::mbar_init(&empty[s], 4);
    }
    dev::fence_mbar_init();
  }
  __syncthreads();
  if (warp == 4) {
    if (lane == 0) {
      const uint64_t policy = dev::policy_evict_first();
      int s = 0;
      uint32_t ph = 0;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!dev::mbar_wait_relaxed(&empty[s], ph ^ 1, status, 41)) break;
        uint8_t* st = smem + s * kStage;
        dev::mbar_expect_tx(&full[s], kWBytes + MT * 8 * BK * 2);
        dev::tma_load_2d_hint(st, &wmap, &full[s], n0, kb * BK, policy);
        dev::tma_load_2d_hint(st + kWBytes / 2, &wmap, &full[s], n0 + 64, kb * BK, policy);
        dev::tma_load_2d(st + kWBytes, &xmap, &full[s], kb * BK, 0);
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
    return;
  }
  // consumers: warp w owns columns [32w, 32w+32) = box w/2, 16-byte chunks 4(w%2) .. 4(w%2)+3
  const int g8 = lane >> 2, t4 = lane & 3;
  float acc[2][MT][4];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][mt][i] = 0.f;
  // ldmatrix.x4.trans over a [16 k][16 n] block: matrices (k 0-7, n 0-7), (k 0-7, n 8-15),
  // (k 8-15, n 0-7), (k 8-15, n 8-15) -> a0..a3 of the 16(n) x 16(k) operand
  const int lrow = (lane & 7) + ((lane >> 4) << 3);  // k row inside the 16-k slab
  const int lchunk = (lane >> 3) & 1;                // which 8-column half of the 16 columns
  int s = 0;
  uint32_t ph = 0;
  for (int kb = 0; kb < kblocks; ++kb) {
    if (!dev::mbar_wait_relaxed_warp(&full[s], ph, status, 42)) return;
    const uint32_t st = dev::smem_u32(smem + s * kStage);
    const uint32_t wbase = st + (warp >> 1) * (kWBytes / 2);
    const uint32_t xbase = st + kWBytes;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      // activations: B fragment b0 = x[m = g8][k = 16 ks + 2 t4 .. +1], b1 = same + 8
      uint32_t xb[MT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        // the activation tile is swizzled like the weights: 16-byte chunk c of row m sits at c ^ (m & 7)
        const uint32_t xrow = xbase + (mt * 8 + g8) * (BK * 2) + t4 * 4;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(xb[mt][0]) : "r"(xrow + (((2 * ks) ^ g8) << 4)));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(xb[mt][1]) : "r"(xrow + (((2 * ks + 1) ^ g8) << 4)));
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int krow = ks * 16 + lrow;
        const int chunk = (warp & 1) * 4 + j * 2 + lchunk;
        uint32_t a[4];
        ldsm_x4_trans(wbase + krow * 128 + ((chunk ^ (krow & 7)) << 4), a);
        // matrices arrive as (k lo, n lo), (k lo, n hi), (k hi, n lo), (k hi, n hi); the MMA wants
        // a0 = (n lo, k lo), a1 = (n hi, k lo), a2 = (n lo, k hi), a3 = (n hi, k hi): same order
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma_bf16(acc[j][mt], a, xb[mt][0], xb[mt][1]);
      }
    }
    __syncwarp();
    if (lane == 0) dev::mbar_arrive(&empty[s]);
    if (++s == kStages) { s = 0; ph ^= 1; }
  }
  // D fragment: d0,d1 = (n = g8, m = 2 t4, 2 t4 + 1), d2,d3 = (n = g8 + 8, same m)
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n0 + warp * 32 + j * 16 + g8 + ((i >> 1) << 3);
        const int m = mt * 8 + 2 * t4 + (i & 1);
        if (m < M && n < N) y[static_cast<size_t>(m) * N + n] = dev::float_to_bf16_bits(acc[j][mt][i]);
      }
}
}  // namespace gemv

}  // namespace dec
}  // namespace qmm

extern "C" {

int qmm_take_rows_bf16(const uint16_t* table, const int32_t* ids, uint16_t* out, int64_t V, int64_t D,
                       int64_t B, uint16_t fill_bits, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(table && ids && out, QMM_ERR_INVALID_ARGUMENT, "qmm_take_rows_bf16: null pointer");
  QMM_REQUIRE(V > 0 && D > 0 && D % 8 == 0 && B >= 0 && V < (1ll << 31), QMM_ERR_INVALID_ARGUMENT,
              "qmm_take_rows_bf16: bad shape (D must be a multiple of 8)");
  QMM_REQUIRE(aligned(table, 16) && aligned(out, 16), QMM_ERR_INVALID_ARGUMENT, "qmm_take_rows_bf16: 16-byte alignment");
  if (B == 0) return QMM_OK;
  QMM_CUDA_TRY(launch_pdl(dec::take_rows_kernel, dim3((unsigned)B), dim3(256), 0, (cudaStream_t)stream, table, ids, out,
                          (int)V, (int)D, fill_bits));
  return QMM_OK;
}

int qmm_add_rmsnorm_bf16(const uint16_t* x, const uint16_t* residual, const uint16_t* weight, uint16_t* sum_out,
                         uint16_t* norm_out, int64_t B, int64_t D, float eps, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(x && weight && norm_out, QMM_ERR_INVALID_ARGUMENT, "qmm_add_rmsnorm_bf16: null pointer");
  QMM_REQUIRE(B >= 0 && D > 0 && D % 2 == 0 && D <= 16384, QMM_ERR_UNSUPPORTED,
              "qmm_add_rmsnorm_bf16: D must be even and <= 16384");
  if (B == 0) return QMM_OK;
  QMM_CUDA_TRY(launch_pdl(dec::add_rmsnorm_kernel, dim3((unsigned)B), dim3(dec::kNormThreads), 0, (cudaStream_t)stream, x,
                          residual, weight, sum_out, norm_out, (int)D, eps));
  return QMM_OK;
}

int qmm_rope_bf16(uint16_t* q, uint16_t* k, const int32_t* positions, int64_t B, int64_t Hq, int64_t Hkv,
                  int64_t head_dim, float theta, int64_t q_ld, int64_t k_ld, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(q && k && positions, QMM_ERR_INVALID_ARGUMENT, "qmm_rope_bf16: null pointer");
  QMM_REQUIRE(B >= 0 && Hq > 0 && Hkv > 0 && head_dim > 0 && head_dim % 2 == 0 && q_ld >= Hq * head_dim &&
                  k_ld >= Hkv * head_dim && B * (Hq + Hkv) * head_dim < (1ll << 31),
              QMM_ERR_INVALID_ARGUMENT, "qmm_rope_bf16: bad shape");
  if (B == 0) return QMM_OK;
  const long long threads = B * (Hq + Hkv) * (head_dim / 2);
  QMM_CUDA_TRY(launch_pdl(dec::rope_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                          q, k, positions, (int)B, (int)Hq, (int)Hkv, (int)head_dim, theta, (long long)q_ld,
                          (long long)k_ld));
  return QMM_OK;
}

int qmm_silu_mul_bf16(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t B, int64_t F, int64_t ld_in,
                      void* stream) {
  using namespace qmm;
  QMM_REQUIRE(gate && up && out, QMM_ERR_INVALID_ARGUMENT, "qmm_silu_mul_bf16: null pointer");
  QMM_REQUIRE(B >= 0 && F > 0 && F % 2 == 0 && ld_in >= F && ld_in % 2 == 0 && B <= 65535, QMM_ERR_INVALID_ARGUMENT,
              "qmm_silu_mul_bf16: bad shape");
  if (B == 0) return QMM_OK;
  dim3 grid((unsigned)((F / 2 + 255) / 256), (unsigned)B);
  QMM_CUDA_TRY(launch_pdl(dec::silu_mul_kernel, grid, dim3(256), 0, (cudaStream_t)stream, gate, up, out, (int)F,
                          (long long)ld_in));
  return QMM_OK;
}

namespace qmm {
namespace dec {
// Splits per (b, kv head): enough CTAs to put two on every SM, at most one per tile.
static int attn_splits(int64_t B, int64_t Hkv, int64_t L) {
  const int64_t ntiles = (L + kTileRows - 1) / kTileRows;
  if (ntiles <= 0) return 0;
  int64_t want = (2 * static_cast<int64_t>(num_sms())) / (B * Hkv);
  if (want < 1) want = 1;
  return static_cast<int>(want < ntiles ? want : ntiles);
}
}  // namespace dec
}  // namespace qmm

size_t qmm_attention_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t L) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || L < 0 || Hq % Hkv) return 0;
  const int nsplit = qmm::dec::attn_splits(B, Hkv, L);
  return static_cast<size_t>(B * Hq * (nsplit > 0 ? nsplit : 1)) * (qmm::dec::kHd + 2) * sizeof(float);
}

int qmm_attention_decode_bf16(const uint16_t* q, const uint16_t* kcache, const uint16_t* vcache,
                              const uint16_t* knew, const uint16_t* vnew, uint16_t* out, int64_t B, int64_t Hq,
                              int64_t Hkv, int64_t L, int64_t head_dim, float scale, int64_t q_ld, int64_t new_ld,
                              void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  using namespace qmm;
  using namespace qmm::dec;
  QMM_REQUIRE(q && knew && vnew && out && (L == 0 || (kcache && vcache)), QMM_ERR_INVALID_ARGUMENT,
              "qmm_attention_decode_bf16: null pointer");
  QMM_REQUIRE(head_dim == kHd, QMM_ERR_UNSUPPORTED, "qmm_attention_decode_bf16: head_dim must be 128");
  QMM_REQUIRE(B > 0 && Hkv > 0 && Hq % Hkv == 0 && L >= 0 && B * Hkv <= 65535 && B * Hkv * L < (1ll << 31),
              QMM_ERR_INVALID_ARGUMENT, "qmm_attention_decode_bf16: bad shape");
  QMM_REQUIRE(q_ld >= Hq * kHd && new_ld >= Hkv * kHd && q_ld % 2 == 0 && aligned(q, 4), QMM_ERR_INVALID_ARGUMENT,
              "qmm_attention_decode_bf16: q_ld / new_ld smaller than a row, or q not 4-byte aligned");
  const int R = static_cast<int>(Hq / Hkv);
  QMM_REQUIRE(R >= 1 && R <= 8, QMM_ERR_UNSUPPORTED,
              "qmm_attention_decode_bf16: %d query heads per kv head (supported: 1 to 8)", R);
  const int nsplit = attn_splits(B, Hkv, L);
  const size_t need = qmm_attention_decode_workspace_bytes(B, Hq, Hkv, L);
  QMM_REQUIRE(workspace && workspace_bytes >= need, QMM_ERR_WORKSPACE,
              "qmm_attention_decode_bf16: %zu bytes of workspace required", need);
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* part = static_cast<float*>(workspace);
  if (nsplit > 0) {
    QMM_REQUIRE(aligned(kcache, 16) && aligned(vcache, 16), QMM_ERR_INVALID_ARGUMENT,
                "qmm_attention_decode_bf16: the cache must be 16-byte aligned");
    CUtensorMap kmap, vmap;
    const uint64_t rows = static_cast<uint64_t>(B * Hkv * L);
    if (int rc = make_tensor_map_2d(&kmap, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, kHd, kHd * 2, kTileRows,
                                    64, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
    if (int rc = make_tensor_map_2d(&vmap, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, kHd, kHd * 2, kTileRows,
                                    64, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
    static std::atomic<uint64_t> configured{0};  // per device
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_partial_kernel), kAttnSmem, configured)) return rc;
    dim3 grid(nsplit, static_cast<unsigned>(B * Hkv));
    QMM_CUDA_TRY(launch_pdl(attn_partial_kernel, grid, dim3(kAttnThreads), kAttnSmem, s, kmap, vmap, q, part, (int)Hq,
                            (int)Hkv, R, (int)L, nsplit, scale, (long long)q_ld,
                            (flags & QMM_ATTN_STATIC_CACHE) ? 1 : 0, device_status_word()));
  }
  QMM_CUDA_TRY(launch_pdl(attn_combine_kernel, dim3(static_cast<unsigned>(B * Hq)), dim3(128), 0, s, part, q, knew, vnew,
                          out, (int)Hq, (int)Hkv, R, nsplit, scale, (long long)q_ld, (long long)new_ld));
  return QMM_OK;
}

int qmm_bf16_matmul_small_m(const uint16_t* x, const uint16_t* w, uint16_t* y, int64_t M, int64_t N, int64_t K,
                            void* stream) {
  using namespace qmm;
  using namespace qmm::dec::gemv;
  QMM_REQUIRE(x && w && y, QMM_ERR_INVALID_ARGUMENT, "qmm_bf16_matmul_small_m: null pointer");
  QMM_REQUIRE(M >= 1 && M <= 16, QMM_ERR_UNSUPPORTED, "qmm_bf16_matmul_small_m: covers 1 <= M <= 16, got %lld",
              (long long)M);
  QMM_REQUIRE(N >= 64 && N % 64 == 0 && K >= BK && K % BK == 0 && N < (1ll << 30) && K < (1ll << 30),
              QMM_ERR_UNSUPPORTED, "qmm_bf16_matmul_small_m: N and K must be positive multiples of 64");
  QMM_REQUIRE(aligned(x, 16) && aligned(w, 16), QMM_ERR_INVALID_ARGUMENT, "qmm_bf16_matmul_small_m: 16-byte alignment");
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  CUtensorMap wmap, xmap;
  if (int rc = make_tensor_map_2d(&wmap, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)N * 2,
                                  BK, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  const int MT = M <= 8 ? 1 : 2;
  if (int rc = make_tensor_map_2d(&xmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)K * 2,
                                  MT * 8, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  static std::atomic<uint64_t> configured1{0}, configured2{0};  // per device
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(bf16_small_m_kernel<1>), kSmem, configured1)) return rc;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(bf16_small_m_kernel<2>), kSmem, configured2)) return rc;
  const unsigned grid = static_cast<unsigned>((N + BN - 1) / BN);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (MT == 1)
    QMM_CUDA_TRY(launch_pdl(bf16_small_m_kernel<1>, dim3(grid), dim3(160), kSmem, s, wmap, xmap, y, (int)M, (int)N, (int)K,
                            device_status_word()));
  else
    QMM_CUDA_TRY(launch_pdl(bf16_small_m_kernel<2>, dim3(grid), dim3(160), kSmem, s, wmap, xmap, y, (int)M, (int)N, (int)K,
                            device_status_word()));
  return QMM_OK;
}

}  // extern "C"
