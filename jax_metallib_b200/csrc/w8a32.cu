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

constexpr int TM = 32, TN = 32, KC = 64;  // tile and k-chunk staged per iteration
constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads)
w8a32_kernel(const float* __restrict__ x, const int8_t* __restrict__ w,
             const float* __restrict__ scale, float* __restrict__ y, int M, int N, int K,
             int k_per_cta) {
  cg::cluster_group cluster = cg::this_cluster();
  const int ks = cluster.block_rank();       // k-slice of this CTA
  const int KS = cluster.num_blocks();
  __shared__ __align__(16) float xs[KC][TM];  // transposed: xs[k][m]
  __shared__ float wsm[KC][TN + 1];
  __shared__ __align__(16) float part[TM][TN];

  const int n0 = blockIdx.x * TN, m0 = blockIdx.y * TM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_begin = ks * k_per_cta;
  const int k_end = min(K, k_begin + k_per_cta);

  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  for (int k0 = k_begin; k0 < k_end; k0 += KC) {
    // stage x (transposed) and w (converted to f32); out-of-range -> 0
    for (int idx = threadIdx.x; idx < TM * KC; idx += kThreads) {
      const int m = idx / KC, kk = idx % KC;
      const int gm = m0 + m, gk = k0 + kk;
      xs[kk][m] = (gm < M && gk < k_end) ? __ldg(x + static_cast<size_t>(gm) * K + gk) : 0.f;
    }
    for (int idx = threadIdx.x; idx < KC * TN; idx += kThreads) {
      const int kk = idx / TN, n = idx % TN;
      const int gk = k0 + kk, gn = n0 + n;
      wsm[kk][n] = (gk < k_end && gn < N)
                       ? static_cast<float>(__ldg(w + static_cast<size_t>(gk) * N + gn))
                       : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < KC; ++kk) {
      const float wv = wsm[kk][lane];
      const float4 a = *reinterpret_cast<const float4*>(&xs[kk][warp * 8]);
      const float4 b = *reinterpret_cast<const float4*>(&xs[kk][warp * 8 + 4]);
      acc[0] = fmaf(a.x, wv, acc[0]);
      acc[1] = fmaf(a.y, wv, acc[1]);
      acc[2] = fmaf(a.z, wv, acc[2]);
      acc[3] = fmaf(a.w, wv, acc[3]);
      acc[4] = fmaf(b.x, wv, acc[4]);
      acc[5] = fmaf(b.y, wv, acc[5]);
      acc[6] = fmaf(b.z, wv, acc[6]);
      acc[7] = fmaf(b.w, wv, acc[7]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[warp * 8 + i][lane] = acc[i];
  cluster.sync();
  if (ks == 0) {
    const int gn = n0 + lane;
    const float sc = (gn < N) ? __ldg(scale + gn) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = warp * 8 + i;
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
  while (KS < 8 && static_cast<long long>(gx) * gy * KS < target && K / (KS * 2) >= KC) KS *= 2;
  int k_per_cta = static_cast<int>((K + KS - 1) / KS);
  k_per_cta = (k_per_cta + KC - 1) / KC * KC;
  if (k_per_cta == 0) k_per_cta = KC;

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
