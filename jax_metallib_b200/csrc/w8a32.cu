// Weight-only int8 (per-output-channel scale) matmul with f32 activations.
//
//   y[M,N] = (x[M,K] @ float(w[K,N])) * scale[N]
//
// Exact f32 FMA arithmetic (int8 -> f32 is exact; the scale is applied once
// per output element instead of once per weight, which differs from the
// un-fused order only by f32 rounding of the product).  At the sizes this is
// called with (a few rows, ~1 MB of weights) the kernel is launch-latency
// bound, so the design goal is many CTAs and no second launch: a 32x32 output
// tile is computed by a thread-block cluster of KS CTAs that split K, and the
// cluster's first CTA adds the partial tiles over distributed shared memory in
// a fixed order (deterministic, no workspace, no atomics).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace qmm {
namespace w8a32 {

constexpr int TM = 32, TN = 32;
constexpr int KC = 256;  // k staged per pass: one global round trip per 256 k
constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
w8a32_kernel(const float* __restrict__ x, const int8_t* __restrict__ w,
             const float* __restrict__ scale, float* __restrict__ y, int M, int N, int K,
             int k_per_cta) {
  cg::cluster_group cluster = cg::this_cluster();
  const int ks = cluster.block_rank();       // k-slice of this CTA
  const int KS = cluster.num_blocks();
  __shared__ __align__(16) float xs[KC][TM];   // transposed: xs[k][m]
  __shared__ __align__(16) int8_t wsm[KC][TN];
  __shared__ __align__(16) float part[TM][TN];

  const int n0 = blockIdx.x * TN, m0 = blockIdx.y * TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;  // warp: rows 4w..4w+3, lane: column
  const int k_begin = ks * k_per_cta;
  const int k_end = min(K, k_begin + k_per_cta);
  const bool vec_ok = (K % 4 == 0) && (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(w) & 15) == 0);

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = k_begin; k0 < k_end; k0 += KC) {
    // stage x (transposed) and w; everything out of range reads as 0.  All loads of
    // a pass are independent, so the pass costs one memory round trip.
    if (vec_ok) {
      for (int idx = threadIdx.x; idx < TM * (KC / 4); idx += kThreads) {
        const int m = idx % TM, kq = idx / TM;  // lanes along m: conflict-free transposed stores
        const int gm = m0 + m, gk = k0 + 4 * kq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gm < M && gk < k_end) v = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(gm) * K + gk));
        xs[4 * kq + 0][m] = v.x;
        xs[4 * kq + 1][m] = (gk + 1 < k_end) ? v.y : 0.f;
        xs[4 * kq + 2][m] = (gk + 2 < k_end) ? v.z : 0.f;
        xs[4 * kq + 3][m] = (gk + 3 < k_end) ? v.w : 0.f;
      }
      for (int idx = threadIdx.x; idx < KC * (TN / 16); idx += kThreads) {
        const int kk = idx / (TN / 16), h = idx % (TN / 16);
        const int gk = k0 + kk, gn = n0 + 16 * h;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (gk < k_end && gn < N) v = __ldg(reinterpret_cast<const uint4*>(w + static_cast<size_t>(gk) * N + gn));
        *reinterpret_cast<uint4*>(&wsm[kk][16 * h]) = v;
      }
    } else {
      for (int idx = threadIdx.x; idx < TM * KC; idx += kThreads) {
        const int m = idx % TM, kk = idx / TM;
        const int gm = m0 + m, gk = k0 + kk;
        xs[kk][m] = (gm < M && gk < k_end) ? __ldg(x + static_cast<size_t>(gm) * K + gk) : 0.f;
      }
      for (int idx = threadIdx.x; idx < KC * TN; idx += kThreads) {
        const int kk = idx / TN, n = idx % TN;
        const int gk = k0 + kk, gn = n0 + n;
        wsm[kk][n] = (gk < k_end && gn < N) ? __ldg(w + static_cast<size_t>(gk) * N + gn) : static_cast<int8_t>(0);
      }
    }
    __syncthreads();
    const int kmax = min(KC, k_end - k0);
#pragma unroll 8
    for (int kk = 0; kk < kmax; ++kk) {
      const float wv = static_cast<float>(wsm[kk][lane]);
      const float4 a = *reinterpret_cast<const float4*>(&xs[kk][warp * 4]);
      acc[0] = fmaf(a.x, wv, acc[0]);
      acc[1] = fmaf(a.y, wv, acc[1]);
      acc[2] = fmaf(a.z, wv, acc[2]);
      acc[3] = fmaf(a.w, wv, acc[3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) part[warp * 4 + i][lane] = acc[i];
  cluster.sync();
  if (ks == 0) {
    const int gn = n0 + lane;
    const float sc = (gn < N) ? __ldg(scale + gn) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = warp * 4 + i;
      float v = acc[i];
      for (int r = 1; r < KS; ++r) {
        const float* remote = cluster.map_shared_rank(&part[0][0], r);
        v += remote[m * TN + lane];
      }
      const int gm = m0 + m;
      if (gm < M && gn < N) y[static_cast<size_t>(gm) * N + gn] = v * sc;
    }
  }
  cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}

}  // namespace w8a32
}  // namespace qmm

extern "C" int qmm_w8a32_perchannel(const float* x, const int8_t* w, const float* scale, float* y,
                                    int64_t M, int64_t N, int64_t K, void* stream) {
  using namespace qmm;
  using namespace qmm::w8a32;
  QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30),
              QMM_ERR_INVALID_ARGUMENT, "qmm_w8a32_perchannel: bad shape");
  if (M == 0 || N == 0) return QMM_OK;  // empty result: nothing to launch, pointers may be null
  QMM_REQUIRE(x && w && scale && y, QMM_ERR_INVALID_ARGUMENT, "qmm_w8a32_perchannel: null pointer");
  const unsigned gx = static_cast<unsigned>((N + TN - 1) / TN);
  const unsigned gy = static_cast<unsigned>((M + TM - 1) / TM);
  QMM_REQUIRE(gy <= 65535, QMM_ERR_UNSUPPORTED, "qmm_w8a32_perchannel: M too large");
  // split K over a cluster until the grid covers the machine (at most 8 CTAs per cluster)
  int KS = 1;
  const int target = num_sms();
  while (KS < 8 && static_cast<long long>(gx) * gy * KS < target && K / (KS * 2) >= 128) KS *= 2;
  int k_per_cta = static_cast<int>((K + KS - 1) / KS);
  k_per_cta = (k_per_cta + 3) / 4 * 4;  // keeps every k-slice 16-byte aligned for the vector loads
  if (k_per_cta == 0) k_per_cta = 4;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(gx, gy, KS);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = KS;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, w8a32_kernel, x, w, scale, y, static_cast<int>(M),
                                  static_cast<int>(N), static_cast<int>(K), k_per_cta));
  return QMM_OK;
}
