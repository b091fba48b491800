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
#include "common.cuh"

namespace qmm {
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
