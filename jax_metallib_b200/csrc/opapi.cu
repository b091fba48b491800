// Fused dequant-GEMM for the operator-API weight formats (weights stored
// transposed, [N, ...] with K contiguous): affine 4/8-bit with f32 scale+bias
// per group, and the MX modes (mxfp4 / mxfp8 / nvfp4).
//
//   y[m,n] = T( sum_k float(x[m,k]) * dequant(w[n,k]) )        T = f32 or f16
//
// K-contiguous weights suit a GEMV-style kernel: one warp owns an output
// column, each lane decodes 8 consecutive k per step (one 32-bit word of
// 4-bit codes or 8 bytes) and keeps up to 8 activation rows in flight; the
// warp reduces with shuffles.  Arithmetic follows the reference kernels:
// weight = scale * q + bias (affine) or scale * element (MX) in f32, product
// and accumulation in f32, one final cast; NaN codes propagate.
//
// These CUDA-core kernels take any M and f32 or f16 activations.  Decode-sized
// f16 problems (M <= 16) go to the tensor-core kernels instead: the TMA-ring
// kernels of opapi_tc.cu where the shape allows, else affine_tc_kernel below.
#include "common.cuh"

namespace qmm {

// the TMA-ring tensor-core kernel for the affine formats
bool affine_ring_covers(int64_t M, int64_t N, int64_t K, int bits, int64_t gs, int dtype, const void* x, const void* w,
                        const float* scales, const float* biases);
int affine_ring_launch(int bits, const void* x, const void* w, const float* scales, const float* biases, void* y, int64_t M,
                       int64_t N, int64_t K, int64_t gs, void* stream);
bool mx_ring_covers(int64_t M, int64_t N, int64_t K, int mode, int dtype, const void* x, const void* w, const void* scales);
int mx_ring_launch(int mode, const void* x, const void* w, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                   void* stream);

namespace opapi {

constexpr int kWarpsPerBlock = 4;
constexpr int RM = 8;  // activation rows per pass

__device__ __constant__ float kE2M1[16] = {0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
                                           -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

__device__ __forceinline__ float decode_e4m3(uint32_t b) {
  if ((b & 127u) == 127u) return __uint_as_float(0x7FC00000u);
  const __half h = __ushort_as_half(static_cast<unsigned short>((b & 127u) << 7));
  const float v = __half2float(h) * 256.0f;
  return (b & 128u) ? -v : v;
}
__device__ __forceinline__ float decode_e8m0(uint32_t b) {
  if (b == 0xFFu) return __uint_as_float(0x7FC00000u);
  return __uint_as_float(b == 0 ? 0x00400000u : (b << 23));
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }

// Decoders: eight dequantised weights for column n, k = k8 .. k8+7.
struct Affine4 {
  const uint32_t* w; const float* s; const float* b; int K; int gs;
  __device__ __forceinline__ void operator()(int n, int k8, float (&o)[8]) const {
    const uint32_t word = __ldg(w + static_cast<size_t>(n) * (K / 8) + k8 / 8);
    const int g = k8 / gs;
    const float sc = __ldg(s + static_cast<size_t>(n) * (K / gs) + g);
    const float bi = __ldg(b + static_cast<size_t>(n) * (K / gs) + g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fmaf(sc, static_cast<float>((word >> (4 * j)) & 0xFu), bi);
  }
};
struct Affine8 {
  const uint8_t* w; const float* s; const float* b; int K; int gs;
  __device__ __forceinline__ void operator()(int n, int k8, float (&o)[8]) const {
    const uint2 words = __ldg(reinterpret_cast<const uint2*>(w + static_cast<size_t>(n) * K + k8));
    const int g = k8 / gs;
    const float sc = __ldg(s + static_cast<size_t>(n) * (K / gs) + g);
    const float bi = __ldg(b + static_cast<size_t>(n) * (K / gs) + g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = fmaf(sc, static_cast<float>((words.x >> (8 * j)) & 0xFFu), bi);
      o[4 + j] = fmaf(sc, static_cast<float>((words.y >> (8 * j)) & 0xFFu), bi);
    }
  }
};
template <int MODE>  // 0 mxfp4 (group 32, e8m0), 1 mxfp8 (group 32, e8m0), 2 nvfp4 (group 16, e4m3)
struct Mx {
  const uint8_t* w; const uint8_t* s; int K;
  __device__ __forceinline__ void operator()(int n, int k8, float (&o)[8]) const {
    constexpr int gs = (MODE == 2) ? 16 : 32;
    const uint32_t sb = __ldg(s + static_cast<size_t>(n) * (K / gs) + k8 / gs);
    const float sc = (MODE == 2) ? decode_e4m3(sb) : decode_e8m0(sb);
    if (MODE == 1) {
      const uint2 words = __ldg(reinterpret_cast<const uint2*>(w + static_cast<size_t>(n) * K + k8));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = sc * decode_e4m3((words.x >> (8 * j)) & 0xFFu);
        o[4 + j] = sc * decode_e4m3((words.y >> (8 * j)) & 0xFFu);
      }
    } else {
      const uint32_t word =
          __ldg(reinterpret_cast<const uint32_t*>(w + static_cast<size_t>(n) * (K / 2) + k8 / 2));
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = sc * kE2M1[(word >> (4 * j)) & 0xFu];
    }
  }
};

template <typename T, typename Dec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qgemm_kernel(const T* __restrict__ x, T* __restrict__ y, Dec dec, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kWarpsPerBlock + warp;
  const int m0 = blockIdx.y * RM;
  if (n >= N) return;
  float acc[RM];
#pragma unroll
  for (int i = 0; i < RM; ++i) acc[i] = 0.f;
  for (int k8 = lane * 8; k8 < K; k8 += 32 * 8) {
    float wv[8];
    dec(n, k8, wv);
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      if (m0 + i < M) {
        float xv[8];
        load8<T>(x + static_cast<size_t>(m0 + i) * K + k8, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    float v = acc[i];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    if (lane == 0 && m0 + i < M) store1(y + static_cast<size_t>(m0 + i) * N + n, v);
  }
}

// ---------------------------------------------------------------------------
// The same arithmetic, laid out for HBM: a warp owns kCols neighbouring output
// columns, every lane fetches 16 bytes of each column's packed row per step (32
// four-bit or 16 eight-bit codes; the next step's words are requested before
// this step is decoded), and an activation chunk read once is used for all
// kCols columns, so the L1 traffic for x is a quarter of the one-column
// kernel's.  E2M1 codes are decoded through a warp shuffle (lane i holds table
// entry i & 15): the constant-memory table of the one-column kernel serialises
// on divergent indices.  Needs K to be a multiple of the codes per 16 bytes and
// 16-byte aligned rows; other shapes take the one-column kernel.
// ---------------------------------------------------------------------------
constexpr int kCols = 4;

__device__ __forceinline__ float u8_to_float(uint32_t v) {  // exact, no I2F
  return __uint_as_float(0x4B000000u | v) - 8388608.f;
}

// Vector decoders: load16(n, k0) fetches the 16 bytes that hold codes k0 .. k0 + kPerLoad - 1 of
// column n; decode8(raw, sub, n, k8, lut, out) turns codes k8 .. k8 + 7 (sub-chunk `sub` of raw)
// into weights.
struct VAffine4 {
  static constexpr int kPerLoad = 32;
  const uint32_t* w; const float* s; const float* b; int K; int gs;
  __device__ __forceinline__ uint4 load16(int n, int k0) const {
    return __ldcs(reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * (K / 8) + k0 / 8));
  }
  __device__ __forceinline__ void decode8(const uint4& raw, int sub, int n, int k8, float, float (&o)[8]) const {
    const uint32_t word = sub == 0 ? raw.x : sub == 1 ? raw.y : sub == 2 ? raw.z : raw.w;
    const int g = k8 / gs;
    const float sc = __ldg(s + static_cast<size_t>(n) * (K / gs) + g);
    const float bi = __ldg(b + static_cast<size_t>(n) * (K / gs) + g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fmaf(sc, u8_to_float((word >> (4 * j)) & 0xFu), bi);
  }
};
struct VAffine8 {
  static constexpr int kPerLoad = 16;
  const uint8_t* w; const float* s; const float* b; int K; int gs;
  __device__ __forceinline__ uint4 load16(int n, int k0) const {
    return __ldcs(reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * K + k0));
  }
  __device__ __forceinline__ void decode8(const uint4& raw, int sub, int n, int k8, float, float (&o)[8]) const {
    const uint32_t w0 = sub == 0 ? raw.x : raw.z, w1 = sub == 0 ? raw.y : raw.w;
    const int g = k8 / gs;
    const float sc = __ldg(s + static_cast<size_t>(n) * (K / gs) + g);
    const float bi = __ldg(b + static_cast<size_t>(n) * (K / gs) + g);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = fmaf(sc, u8_to_float((w0 >> (8 * j)) & 0xFFu), bi);
      o[4 + j] = fmaf(sc, u8_to_float((w1 >> (8 * j)) & 0xFFu), bi);
    }
  }
};
template <int MODE>  // 0 mxfp4, 1 mxfp8, 2 nvfp4
struct VMx {
  static constexpr int kPerLoad = (MODE == 1) ? 16 : 32;
  const uint8_t* w; const uint8_t* s; int K;
  __device__ __forceinline__ uint4 load16(int n, int k0) const {
    const size_t off = (MODE == 1) ? static_cast<size_t>(n) * K + k0 : static_cast<size_t>(n) * (K / 2) + k0 / 2;
    return __ldcs(reinterpret_cast<const uint4*>(w + off));
  }
  __device__ __forceinline__ void decode8(const uint4& raw, int sub, int n, int k8, float lut, float (&o)[8]) const {
    constexpr int gs = (MODE == 2) ? 16 : 32;
    const uint32_t sb = __ldg(s + static_cast<size_t>(n) * (K / gs) + k8 / gs);
    const float sc = (MODE == 2) ? decode_e4m3(sb) : decode_e8m0(sb);
    if (MODE == 1) {
      const uint32_t w0 = sub == 0 ? raw.x : raw.z, w1 = sub == 0 ? raw.y : raw.w;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = sc * decode_e4m3((w0 >> (8 * j)) & 0xFFu);
        o[4 + j] = sc * decode_e4m3((w1 >> (8 * j)) & 0xFFu);
      }
    } else {
      const uint32_t word = sub == 0 ? raw.x : sub == 1 ? raw.y : sub == 2 ? raw.z : raw.w;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o[j] = sc * __shfl_sync(0xFFFFFFFFu, lut, static_cast<int>((word >> (4 * j)) & 0xFu));
    }
  }
};

template <typename T, typename VDec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qgemm_vec_kernel(const T* __restrict__ x, T* __restrict__ y, VDec dec, int M, int N, int K) {
  constexpr int KL = VDec::kPerLoad;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kWarpsPerBlock + warp) * kCols;
  const int m0 = blockIdx.y * RM;
  if (n0 >= N) return;  // whole warp
  const float lut = kE2M1[lane & 15];
  int ncol[kCols];  // columns past N repeat the last one (their results are not stored)
#pragma unroll
  for (int c = 0; c < kCols; ++c) ncol[c] = min(n0 + c, N - 1);
  float acc[kCols][RM];
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int i = 0; i < RM; ++i) acc[c][i] = 0.f;

  const int step = 32 * KL;
  int k0 = lane * KL;
  uint4 raw[kCols], nxt[kCols];
  if (k0 < K) {
#pragma unroll
    for (int c = 0; c < kCols; ++c) raw[c] = dec.load16(ncol[c], k0);
  }
  // All lanes run the same number of iterations (the shuffle inside the decoder needs the whole
  // warp); a lane past the end of K computes on zeros of x.
  const int iters = (K + step - 1) / step;
  for (int it = 0; it < iters; ++it, k0 += step) {
    const bool live = k0 < K;
    const bool more = k0 + step < K;
    if (more) {
#pragma unroll
      for (int c = 0; c < kCols; ++c) nxt[c] = dec.load16(ncol[c], k0 + step);
    }
#pragma unroll
    for (int sub = 0; sub < KL / 8; ++sub) {
      const int k8 = live ? k0 + sub * 8 : 0;
      float wv[kCols][8];
#pragma unroll
      for (int c = 0; c < kCols; ++c) dec.decode8(live ? raw[c] : make_uint4(0, 0, 0, 0), sub, ncol[c], k8, lut, wv[c]);
      if (live) {
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          if (m0 + i < M) {
            float xv[8];
            load8<T>(x + static_cast<size_t>(m0 + i) * K + k8, xv);
#pragma unroll
            for (int c = 0; c < kCols; ++c)
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[c][i] = fmaf(xv[j], wv[c][j], acc[c][i]);
          }
        }
      }
    }
    if (more) {
#pragma unroll
      for (int c = 0; c < kCols; ++c) raw[c] = nxt[c];
    }
  }
#pragma unroll
  for (int c = 0; c < kCols; ++c)
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      float v = acc[c][i];
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
      if (lane == 0 && m0 + i < M && n0 + c < N) store1(y + static_cast<size_t>(m0 + i) * N + n0 + c, v);
    }
}

// ---------------------------------------------------------------------------
// Tensor-core route for the affine formats at decode sizes (f16 activations, M <= 16, group_size a
// multiple of the 64 (4-bit) or 32 (8-bit) k that a quad of threads covers per step).  The CUDA-core
// kernels above spend about nine lane instructions per weight, several times what the memory
// system needs to keep up; here a weight costs a fraction of one:
//   sum_k x[m,k] * (s * q[n,k] + b) = s * sum_k x q + b * sum_k x        per (n, group)
// so the packed words go to mma.sync.m16n8k16 as they are.  A shift and an AND leave two codes of a
// word in the low bits of the two halves of a register, where each reads as the f16 subnormal
// q * 2^-24 (exact for q < 1024); the factor 2^24 is folded into the group's scale.  The 16 rows of
// the MMA's first operand are 16 output columns (a thread holds two of them), its 16 k-slots are
// four codes of one packed word per thread of a quad, and the activations are staged in shared
// memory once per CTA in exactly that slot order, so a thread's fragments are one 8-byte load per
// weight row and 16-byte shared loads of activations.  A CTA has eight warps: four 16-column tiles
// times two halves of K, combined through shared memory.  sum_k x per (row, group) is computed once
// per CTA.  Products are exact (f16 x f16 in f32), accumulation is f32; the scale and bias are
// applied per group instead of per weight, which moves the result by f32 rounding only.
// ---------------------------------------------------------------------------
namespace tcq {
constexpr int kThreads = 256;
constexpr int kTileCols = 16;
constexpr int kTilesPerCta = 4;
constexpr int kDepth = 8;  // steps of weights in flight per thread (8 bytes per row and step)
constexpr int kMaxSmem = 200 * 1024;

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int BITS>
struct Fmt {
  static constexpr int kPerWord = 32 / BITS;       // codes per 32-bit word
  static constexpr int kSpan = 8 * kPerWord;       // k per step of a quad: 4 threads x 2 words
  // staged activation rows are padded so that the two rows of a quarter-warp's 16-byte loads fall
  // into different banks: a quad reads 4 x 16 bytes 32 apart (4-bit) or 64 contiguous bytes (8-bit)
  static constexpr int kRowPad = BITS == 4 ? 16 : 64;
};

// bytes of dynamic shared memory: staged activations, sums per (row, group), the hand-over of the
// second K half
template <int BITS>
inline size_t smem_bytes(int MT, int K, int G) {
  return static_cast<size_t>(MT) * 8 * (static_cast<size_t>(K) * 2 + Fmt<BITS>::kRowPad) +
         static_cast<size_t>(MT) * 8 * G * 4 + static_cast<size_t>(kTilesPerCta) * 32 * MT * 4 * 4;
}

template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads)
affine_tc_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ w, const float* __restrict__ scales,
                 const float* __restrict__ biases, __half* __restrict__ y, int M, int N, int K, int gs) {
  using F = Fmt<BITS>;
  extern __shared__ __align__(16) uint8_t smem[];
  const int G = K / gs;
  const int row_bytes = K * 2 + F::kRowPad;
  uint8_t* xs = smem;
  float* xsum = reinterpret_cast<float*>(smem + static_cast<size_t>(MT) * 8 * row_bytes);
  float* hand = xsum + MT * 8 * G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- stage the activations in MMA slot order.  Per 8 k (16 bytes):
  //   4-bit (one word):  (x0,x4) (x1,x5) (x2,x6) (x3,x7)
  //   8-bit (two words): (x0,x2) (x1,x3) (x4,x6) (x5,x7)
  const int chunks = K / 8;
  for (int i = tid; i < MT * 8 * chunks; i += kThreads) {
    const int m = i / chunks, c8 = i - m * chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < M) v = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * K + c8 * 8));
    const uint32_t h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;  // (x0,x1) (x2,x3) (x4,x5) (x6,x7)
    uint4 o;
    if (BITS == 4) {
      o.x = __byte_perm(h0, h2, 0x5410);
      o.y = __byte_perm(h0, h2, 0x7632);
      o.z = __byte_perm(h1, h3, 0x5410);
      o.w = __byte_perm(h1, h3, 0x7632);
    } else {
      o.x = __byte_perm(h0, h1, 0x5410);
      o.y = __byte_perm(h0, h1, 0x7632);
      o.z = __byte_perm(h2, h3, 0x5410);
      o.w = __byte_perm(h2, h3, 0x7632);
    }
    *reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * row_bytes + c8 * 16) = o;
  }
  for (int i = tid; i < MT * 8 * G; i += kThreads) {  // one thread per (row, group): a fixed summation order
    const int m = i / G, g = i - m * G;
    float acc = 0.f;
    if (m < M)
      for (int k = 0; k < gs; k += 8) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * K + g * gs + k));
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          acc += f.x + f.y;
        }
      }
    xsum[m * G + g] = acc;
  }
  __syncthreads();

  const int tile = warp & 3, khalf = warp >> 2;
  const int n0 = (blockIdx.x * kTilesPerCta + tile) * kTileCols;
  const int g8 = lane >> 2, t4 = lane & 3;
  float yacc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;

  if (n0 < N) {  // whole warp; N is a multiple of 16, so the tile is complete
    const int g_begin = khalf == 0 ? 0 : (G + 1) / 2, g_end = khalf == 0 ? (G + 1) / 2 : G;
    const int steps_per_group = gs / F::kSpan;
    const int total = (g_end - g_begin) * steps_per_group;
    const int words_per_row = K / F::kPerWord;
    const int word_begin = g_begin * (gs / F::kPerWord) + 2 * t4;  // this thread's first word within a row
    const uint32_t* w0 = w + static_cast<size_t>(n0 + g8) * words_per_row + word_begin;
    const uint32_t* w1 = w0 + static_cast<size_t>(8) * words_per_row;
    const float* s0 = scales + static_cast<size_t>(n0 + g8) * G, *s1 = s0 + static_cast<size_t>(8) * G;
    const float* b0p = biases + static_cast<size_t>(n0 + g8) * G, *b1p = b0p + static_cast<size_t>(8) * G;
    // a word's activations: 16 staged bytes (4-bit) or 8 (8-bit)
    const uint8_t* xrow = xs + static_cast<size_t>(g8) * row_bytes + static_cast<size_t>(word_begin) * (2 * F::kPerWord);
    constexpr int kStepXBytes = 8 * 2 * F::kPerWord;  // staged bytes a step of 8 words advances
    uint2 qa[kDepth], qb[kDepth];  // steps in flight: two words of row g8, two of row g8 + 8
#pragma unroll
    for (int i = 0; i < kDepth; ++i)
      if (i < total) {
        qa[i] = __ldcs(reinterpret_cast<const uint2*>(w0 + i * 8));
        qb[i] = __ldcs(reinterpret_cast<const uint2*>(w1 + i * 8));
      }
    float d[MT][4];
    int in_group = 0, g = g_begin;
    for (int base = 0; base < total; base += kDepth) {
#pragma unroll
      for (int i = 0; i < kDepth; ++i) {
        const int sp = base + i;
        if (sp >= total) break;
        if (in_group == 0) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) d[mt][j] = 0.f;
        }
        const uint2 a = qa[i], b = qb[i];
        if (sp + kDepth < total) {  // refill the slot
          qa[i] = __ldcs(reinterpret_cast<const uint2*>(w0 + (sp + kDepth) * 8));
          qb[i] = __ldcs(reinterpret_cast<const uint2*>(w1 + (sp + kDepth) * 8));
        }
        if (BITS == 4) {
          constexpr uint32_t kNib = 0x000F000Fu;
#pragma unroll
          for (int wi = 0; wi < 2; ++wi) {
            const uint32_t lo = wi ? a.y : a.x, hi = wi ? b.y : b.x;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xq = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(mt) * 8 * row_bytes +
                                                               static_cast<size_t>(sp) * kStepXBytes + wi * 16);
              mma16816(d[mt], lo & kNib, hi & kNib, (lo >> 4) & kNib, (hi >> 4) & kNib, xq.x, xq.y);
              mma16816(d[mt], (lo >> 8) & kNib, (hi >> 8) & kNib, (lo >> 12) & kNib, (hi >> 12) & kNib, xq.z, xq.w);
            }
          }
        } else {
          constexpr uint32_t kByte = 0x00FF00FFu;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xq = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(mt) * 8 * row_bytes +
                                                             static_cast<size_t>(sp) * kStepXBytes);
            mma16816(d[mt], a.x & kByte, b.x & kByte, (a.x >> 8) & kByte, (b.x >> 8) & kByte, xq.x, xq.y);
            mma16816(d[mt], a.y & kByte, b.y & kByte, (a.y >> 8) & kByte, (b.y >> 8) & kByte, xq.z, xq.w);
          }
        }
        if (++in_group == steps_per_group) {
          in_group = 0;
          const float sc0 = __ldg(s0 + g) * 16777216.f, sc1 = __ldg(s1 + g) * 16777216.f;
          const float bi0 = __ldg(b0p + g), bi1 = __ldg(b1p + g);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float xs0 = xsum[(mt * 8 + 2 * t4) * G + g], xs1 = xsum[(mt * 8 + 2 * t4 + 1) * G + g];
            yacc[mt][0] = fmaf(bi0, xs0, fmaf(sc0, d[mt][0], yacc[mt][0]));
            yacc[mt][1] = fmaf(bi0, xs1, fmaf(sc0, d[mt][1], yacc[mt][1]));
            yacc[mt][2] = fmaf(bi1, xs0, fmaf(sc1, d[mt][2], yacc[mt][2]));
            yacc[mt][3] = fmaf(bi1, xs1, fmaf(sc1, d[mt][3], yacc[mt][3]));
          }
          ++g;
        }
      }
    }
  }
  // ---- the second K half hands its sums to the first, which stores
  float* slot = hand + (tile * 32 + lane) * MT * 4;
  if (khalf == 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) slot[mt * 4 + i] = yacc[mt][i];
  }
  __syncthreads();
  if (khalf == 0 && n0 < N) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n0 + g8 + ((i >> 1) << 3), m = mt * 8 + 2 * t4 + (i & 1);
        if (m < M) y[static_cast<size_t>(m) * N + n] = __float2half_rn(yacc[mt][i] + slot[mt * 4 + i]);
      }
    }
  }
}

template <int BITS, int MT>
static int launch_one(const void* x, const void* w, const float* scales, const float* biases, void* y, int64_t M,
                      int64_t N, int64_t K, int64_t gs, void* stream) {
  static std::atomic<uint64_t> configured{0};
  auto kernel = affine_tc_kernel<BITS, MT>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxSmem, configured)) return rc;
  const size_t smem = smem_bytes<BITS>(MT, static_cast<int>(K), static_cast<int>(K / gs));
  const unsigned grid = static_cast<unsigned>((N + kTileCols * kTilesPerCta - 1) / (kTileCols * kTilesPerCta));
  kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(x), static_cast<const uint32_t*>(w), scales, biases, static_cast<__half*>(y),
      static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), static_cast<int>(gs));
  QMM_CHECK_LAUNCH(BITS == 4 ? "affine_qgemm_4bit_f16 (tensor cores)" : "affine_qgemm_8bit_f16 (tensor cores)");
  return QMM_OK;
}

static int launch(int bits, const void* x, const void* w, const float* scales, const float* biases, void* y, int64_t M,
                  int64_t N, int64_t K, int64_t gs, void* stream) {
  if (bits == 4)
    return M <= 8 ? launch_one<4, 1>(x, w, scales, biases, y, M, N, K, gs, stream)
                  : launch_one<4, 2>(x, w, scales, biases, y, M, N, K, gs, stream);
  return M <= 8 ? launch_one<8, 1>(x, w, scales, biases, y, M, N, K, gs, stream)
                : launch_one<8, 2>(x, w, scales, biases, y, M, N, K, gs, stream);
}

// shapes the tensor-core route covers
static bool covers(int64_t M, int64_t N, int64_t K, int bits, int64_t gs, int dtype, const void* x, const void* w) {
  if ((bits != 4 && bits != 8) || dtype != QMM_F16 || M < 1 || M > 16 || N % 16 != 0) return false;
  const int span = bits == 4 ? Fmt<4>::kSpan : Fmt<8>::kSpan;
  if (gs % span != 0 || K % gs != 0 || K > (1 << 20)) return false;
  if (!aligned(x, 16) || !aligned(w, 8)) return false;
  const int MT = M <= 8 ? 1 : 2;
  const size_t smem = bits == 4 ? smem_bytes<4>(MT, static_cast<int>(K), static_cast<int>(K / gs))
                                : smem_bytes<8>(MT, static_cast<int>(K), static_cast<int>(K / gs));
  return smem <= static_cast<size_t>(kMaxSmem);
}
}  // namespace tcq

template <typename T, typename VDec>
static int launch_vec(const void* x, void* y, VDec dec, int64_t M, int64_t N, int64_t K, void* stream,
                      const char* name) {
  dim3 grid(static_cast<unsigned>((N + kWarpsPerBlock * kCols - 1) / (kWarpsPerBlock * kCols)),
            static_cast<unsigned>((M + RM - 1) / RM));
  QMM_REQUIRE(grid.y <= 65535, QMM_ERR_UNSUPPORTED, "%s: M too large", name);
  qgemm_vec_kernel<T, VDec><<<grid, kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const T*>(x), static_cast<T*>(y), dec, static_cast<int>(M), static_cast<int>(N),
      static_cast<int>(K));
  QMM_CHECK_LAUNCH(name);
  return QMM_OK;
}

template <typename T, typename Dec>
static int launch(const void* x, void* y, Dec dec, int64_t M, int64_t N, int64_t K, void* stream,
                  const char* name) {
  if (M == 0 || N == 0) return QMM_OK;
  dim3 grid(static_cast<unsigned>((N + kWarpsPerBlock - 1) / kWarpsPerBlock),
            static_cast<unsigned>((M + RM - 1) / RM));
  QMM_REQUIRE(grid.y <= 65535, QMM_ERR_UNSUPPORTED, "%s: M too large", name);
  qgemm_kernel<T, Dec><<<grid, kWarpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const T*>(x), static_cast<T*>(y), dec, static_cast<int>(M), static_cast<int>(N),
      static_cast<int>(K));
  QMM_CHECK_LAUNCH(name);
  return QMM_OK;
}

}  // namespace opapi
}  // namespace qmm

extern "C" {

int qmm_affine_matmul(const void* x, const void* w_packed, const float* scales, const float* biases,
                      void* y, int64_t M, int64_t N, int64_t K, int bits, int64_t group_size,
                      int dtype, void* stream) {
  using namespace qmm;
  using namespace qmm::opapi;
  QMM_REQUIRE(x && w_packed && scales && biases && y, QMM_ERR_INVALID_ARGUMENT,
              "qmm_affine_matmul: null pointer");
  QMM_REQUIRE(bits == 4 || bits == 8, QMM_ERR_UNSUPPORTED,
              "qmm_affine_matmul: fused kernels exist for bits 4 and 8, got %d", bits);
  QMM_REQUIRE(dtype == QMM_F32 || dtype == QMM_F16, QMM_ERR_UNSUPPORTED,
              "qmm_affine_matmul: activations must be float32 or float16");
  QMM_REQUIRE(M >= 0 && N >= 0 && K > 0 && K < (1ll << 30) && N < (1ll << 30) && M < (1ll << 30),
              QMM_ERR_INVALID_ARGUMENT, "qmm_affine_matmul: bad shape");
  QMM_REQUIRE(group_size > 0 && group_size % 8 == 0 && K % group_size == 0, QMM_ERR_INVALID_ARGUMENT,
              "qmm_affine_matmul: K (%lld) must be divisible by group_size (%lld), a multiple of 8",
              (long long)K, (long long)group_size);
  QMM_REQUIRE(aligned(x, 16) && aligned(w_packed, 8), QMM_ERR_INVALID_ARGUMENT,
              "qmm_affine_matmul: x must be 16-byte and w_packed 8-byte aligned");
  const int k = static_cast<int>(K), gs = static_cast<int>(group_size);
  if (M == 0 || N == 0) return QMM_OK;
  // decode-sized f16 problems: the tensor-core kernels (TMA ring where the shape allows, else plain loads)
  if (affine_ring_covers(M, N, K, bits, group_size, dtype, x, w_packed, scales, biases))
    return affine_ring_launch(bits, x, w_packed, scales, biases, y, M, N, K, group_size, stream);
  if (tcq::covers(M, N, K, bits, group_size, dtype, x, w_packed))
    return tcq::launch(bits, x, w_packed, scales, biases, y, M, N, K, group_size, stream);
  // rows of 16-byte words: the vectorised kernel
  if (aligned(w_packed, 16) && K % (bits == 4 ? 32 : 16) == 0) {
    if (bits == 4) {
      VAffine4 d{static_cast<const uint32_t*>(w_packed), scales, biases, k, gs};
      return dtype == QMM_F32 ? launch_vec<float>(x, y, d, M, N, K, stream, "affine_qgemm_4bit_f32")
                              : launch_vec<__half>(x, y, d, M, N, K, stream, "affine_qgemm_4bit_f16");
    }
    VAffine8 d{static_cast<const uint8_t*>(w_packed), scales, biases, k, gs};
    return dtype == QMM_F32 ? launch_vec<float>(x, y, d, M, N, K, stream, "affine_qgemm_8bit_f32")
                            : launch_vec<__half>(x, y, d, M, N, K, stream, "affine_qgemm_8bit_f16");
  }
  if (bits == 4) {
    Affine4 d{static_cast<const uint32_t*>(w_packed), scales, biases, k, gs};
    return dtype == QMM_F32 ? launch<float>(x, y, d, M, N, K, stream, "affine_qgemm_4bit_f32")
                            : launch<__half>(x, y, d, M, N, K, stream, "affine_qgemm_4bit_f16");
  }
  Affine8 d{static_cast<const uint8_t*>(w_packed), scales, biases, k, gs};
  return dtype == QMM_F32 ? launch<float>(x, y, d, M, N, K, stream, "affine_qgemm_8bit_f32")
                          : launch<__half>(x, y, d, M, N, K, stream, "affine_qgemm_8bit_f16");
}

int qmm_mx_matmul(const void* x, const uint8_t* w_packed, const uint8_t* scales, void* y, int64_t M,
                  int64_t N, int64_t K, int mode, int dtype, void* stream) {
  using namespace qmm;
  using namespace qmm::opapi;
  QMM_REQUIRE(x && w_packed && scales && y, QMM_ERR_INVALID_ARGUMENT, "qmm_mx_matmul: null pointer");
  QMM_REQUIRE(mode == QMM_MXFP4 || mode == QMM_MXFP8 || mode == QMM_NVFP4, QMM_ERR_INVALID_ARGUMENT,
              "qmm_mx_matmul: unknown mode %d", mode);
  QMM_REQUIRE(dtype == QMM_F32 || dtype == QMM_F16, QMM_ERR_UNSUPPORTED,
              "qmm_mx_matmul: activations must be float32 or float16");
  const int64_t gs = (mode == QMM_NVFP4) ? 16 : 32;
  QMM_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % gs == 0 && K < (1ll << 30) && N < (1ll << 30) &&
                  M < (1ll << 30),
              QMM_ERR_INVALID_ARGUMENT, "qmm_mx_matmul: K (%lld) must be a positive multiple of %lld",
              (long long)K, (long long)gs);
  QMM_REQUIRE(aligned(x, 16) && aligned(w_packed, 8), QMM_ERR_INVALID_ARGUMENT,
              "qmm_mx_matmul: x must be 16-byte and w_packed 8-byte aligned");
  const int k = static_cast<int>(K);
  if (M == 0 || N == 0) return QMM_OK;
  static_assert(QMM_MXFP4 == 0 && QMM_MXFP8 == 1 && QMM_NVFP4 == 2, "mode numbering shared with the tensor-core kernel");
  if (mx_ring_covers(M, N, K, mode, dtype, x, w_packed, scales))   // decode-sized f16 problems: the tensor-core kernel
    return mx_ring_launch(mode, x, w_packed, scales, y, M, N, K, stream);
  if (aligned(w_packed, 16) && K % 32 == 0) {  // rows of 16-byte words: the vectorised kernel
    if (mode == QMM_MXFP4) {
      VMx<0> d{w_packed, scales, k};
      return dtype == QMM_F32 ? launch_vec<float>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp4_f32")
                              : launch_vec<__half>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp4_f16");
    }
    if (mode == QMM_MXFP8) {
      VMx<1> d{w_packed, scales, k};
      return dtype == QMM_F32 ? launch_vec<float>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp8_f32")
                              : launch_vec<__half>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp8_f16");
    }
    VMx<2> d{w_packed, scales, k};
    return dtype == QMM_F32 ? launch_vec<float>(x, y, d, M, N, K, stream, "mx_qgemm_nvfp4_f32")
                            : launch_vec<__half>(x, y, d, M, N, K, stream, "mx_qgemm_nvfp4_f16");
  }
  if (mode == QMM_MXFP4) {
    Mx<0> d{w_packed, scales, k};
    return dtype == QMM_F32 ? launch<float>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp4_f32")
                            : launch<__half>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp4_f16");
  }
  if (mode == QMM_MXFP8) {
    Mx<1> d{w_packed, scales, k};
    return dtype == QMM_F32 ? launch<float>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp8_f32")
                            : launch<__half>(x, y, d, M, N, K, stream, "mx_qgemm_mxfp8_f16");
  }
  Mx<2> d{w_packed, scales, k};
  return dtype == QMM_F32 ? launch<float>(x, y, d, M, N, K, stream, "mx_qgemm_nvfp4_f32")
                          : launch<__half>(x, y, d, M, N, K, stream, "mx_qgemm_nvfp4_f16");
}

}  // extern "C"
