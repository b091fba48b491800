// Entry points whose work is routed between the tcgen05 GEMMs and plain
// CUDA-core kernels.  The tensor-core kernels take every shape TMA can
// describe (16-byte row pitches); anything else (the few-element shapes of the
// reference's integer-dot tests, odd strides) runs on the simple kernels below.
// Both routes are GPU code; there is no host fallback.
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace qmm {

int i8gemm_tcgen05(const void* a, const void* b, int32_t* acc, const float* row_scale,
                   const float* col_scale, float* out, int64_t M, int64_t N, int64_t K,
                   int a_unsigned, int b_unsigned, cudaStream_t stream);
int w8a16_tcgen05(const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y, int64_t M,
                  int64_t N, int64_t K, int64_t ldy, uint32_t flags, uint32_t* signal, uint32_t* arrive,
                  cudaStream_t stream);

namespace simple {

template <bool AU, bool BU>
__global__ void i8dot_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b,
                             int32_t* __restrict__ acc, float* __restrict__ out,
                             const float* __restrict__ rs, const float* __restrict__ cs, int M, int N,
                             int K) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y;
  if (n >= N || m >= M) return;
  int32_t s = 0;  // wraps mod 2^32 like the reference's int32 accumulator
  for (int k = 0; k < K; ++k) {
    const int av = AU ? static_cast<int>(a[static_cast<size_t>(m) * K + k])
                      : static_cast<int>(static_cast<int8_t>(a[static_cast<size_t>(m) * K + k]));
    const int bv = BU ? static_cast<int>(b[static_cast<size_t>(k) * N + n])
                      : static_cast<int>(static_cast<int8_t>(b[static_cast<size_t>(k) * N + n]));
    s = static_cast<int32_t>(static_cast<uint32_t>(s) + static_cast<uint32_t>(av * bv));
  }
  if (acc) acc[static_cast<size_t>(m) * N + n] = s;
  if (out) out[static_cast<size_t>(m) * N + n] = static_cast<float>(s) * rs[m] * cs[n];
}

__global__ void w8a16_kernel(const uint16_t* __restrict__ x, const int8_t* __restrict__ w,
                             const float* __restrict__ scale, uint16_t* __restrict__ y, int M, int N,
                             int K, long long ldy) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y;
  if (n >= N || m >= M) return;
  float s = 0.f;
  for (int k = 0; k < K; ++k)
    s = fmaf(dev::bf16_bits_to_float(x[static_cast<size_t>(m) * K + k]),
             static_cast<float>(w[static_cast<size_t>(k) * N + n]), s);
  y[static_cast<size_t>(m) * ldy + n] = dev::float_to_bf16_bits(s * scale[n]);
}

// One thread per word: wait (bounded) until words[i] >= expected.  The words are written by other
// GPUs (the completion signals of a sharded linear), never by a kernel sharing this GPU.
__global__ void wait_words_kernel(const uint32_t* words, int count, uint32_t expected, unsigned long long limit_ns,
                                  int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint64_t t0 = dev::globaltimer_ns();
  while (true) {
    // counts wrap: "reached" means no more than 2^31 behind
    if (static_cast<int32_t>(dev::ld_acquire_sys_u32(words + i) - expected) >= 0) return;
    if (dev::globaltimer_ns() - t0 > limit_ns) break;
    __nanosleep(200);
  }
  if (status) atomicExch(status, (60 << 16) | QMM_ERR_TIMEOUT);
}

// Local block -> multicast address, 16 bytes per thread, four loads in flight per thread; the last CTA to finish
// publishes the completion count on every rank (tag of the bounded wait that reads it: 60).
__global__ void __launch_bounds__(512)
multicast_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst_mc, size_t n16, uint32_t* signal_mc,
                      uint32_t* arrive) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = src[i + j * stride];
#pragma unroll
    for (int j = 0; j < 4; ++j) dev::multimem_st_v4_b32(dst_mc + i + j * stride, v[j]);
  }
  for (; i < n16; i += stride) dev::multimem_st_v4_b32(dst_mc + i, src[i]);
  dev::fence_sys();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicInc(arrive, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      dev::fence_sys();
      dev::multimem_red_release_add_u32(signal_mc, 1u);
    }
  }
}

struct PeerList {
  uint4* dst[QMM_MAX_PEERS];
  uint32_t* signal[QMM_MAX_PEERS];
  int n;
};
// Local block -> the same block of every peer's buffer by plain stores over NVLink (no copy to this GPU).
__global__ void __launch_bounds__(512)
peer_copy_kernel(const uint4* __restrict__ src, PeerList peers, size_t n16, uint32_t* local_signal, uint32_t* arrive) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = src[i + j * stride];
    for (int p = 0; p < peers.n; ++p) {
#pragma unroll
      for (int j = 0; j < 4; ++j) __stcg(peers.dst[p] + i + j * stride, v[j]);
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = src[i];
    for (int p = 0; p < peers.n; ++p) __stcg(peers.dst[p] + i, v);
  }
  dev::fence_sys();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicInc(arrive, gridDim.x - 1);
    if (prev == gridDim.x - 1) {
      dev::fence_sys();
      for (int p = 0; p < peers.n; ++p) dev::red_release_sys_add_u32(peers.signal[p], 1u);
      dev::red_release_sys_add_u32(local_signal, 1u);
    }
  }
}

}  // namespace simple

// QMM_FORCE_SIMPLE=1 routes every shape to the CUDA-core kernels (a cross-check of the tensor-core
// route on a GPU box); read once per process.
static int force_simple() {
  static std::atomic<int> cache{INT32_MIN};
  return env_int_once("QMM_FORCE_SIMPLE", 0, cache);
}

}  // namespace qmm

extern "C" {

int qmm_i8i8_i32(const void* a, const void* b, int32_t* acc, const float* row_scale,
                 const float* col_scale, float* out, int64_t M, int64_t N, int64_t K,
                 int a_unsigned, int b_unsigned, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30),
              QMM_ERR_INVALID_ARGUMENT, "qmm_i8i8_i32: bad shape");
  if (M == 0 || N == 0) return QMM_OK;  // empty result
  QMM_REQUIRE(a && b, QMM_ERR_INVALID_ARGUMENT, "qmm_i8i8_i32: null operand");
  QMM_REQUIRE(acc || out, QMM_ERR_INVALID_ARGUMENT, "qmm_i8i8_i32: neither acc nor out requested");
  QMM_REQUIRE(!out || (row_scale && col_scale), QMM_ERR_INVALID_ARGUMENT,
              "qmm_i8i8_i32: out needs row_scale and col_scale");
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tma_ok = K > 0 && K % 16 == 0 && N % 16 == 0 && aligned(a, 16) && aligned(b, 16) &&
                      (!acc || aligned(acc, 16)) && (!out || (aligned(out, 16) && aligned(col_scale, 16)));
  if (tma_ok && M * N >= 128 * 128 && !force_simple())
    return i8gemm_tcgen05(a, b, acc, row_scale, col_scale, out, M, N, K, a_unsigned, b_unsigned, s);
  QMM_REQUIRE(M <= 65535, QMM_ERR_UNSUPPORTED, "qmm_i8i8_i32: unaligned shape with M > 65535");
  dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(M));
  const uint8_t* ap = static_cast<const uint8_t*>(a);
  const uint8_t* bp = static_cast<const uint8_t*>(b);
  const int m = (int)M, n = (int)N, k = (int)K;
  if (a_unsigned && b_unsigned)
    simple::i8dot_kernel<true, true><<<grid, 128, 0, s>>>(ap, bp, acc, out, row_scale, col_scale, m, n, k);
  else if (a_unsigned)
    simple::i8dot_kernel<true, false><<<grid, 128, 0, s>>>(ap, bp, acc, out, row_scale, col_scale, m, n, k);
  else if (b_unsigned)
    simple::i8dot_kernel<false, true><<<grid, 128, 0, s>>>(ap, bp, acc, out, row_scale, col_scale, m, n, k);
  else
    simple::i8dot_kernel<false, false><<<grid, 128, 0, s>>>(ap, bp, acc, out, row_scale, col_scale, m, n, k);
  QMM_CHECK_LAUNCH("i8dot_kernel");
  return QMM_OK;
}

static int w8a16_entry(const char* name, const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y,
                       int64_t M, int64_t N, int64_t K, int64_t ldy, const qmm_gemm_ext* ext, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30) &&
                  ldy >= N,
              QMM_ERR_INVALID_ARGUMENT, "%s: bad shape (ldy must be >= N)", name);
  uint32_t flags = 0;
  uint32_t* signal = nullptr;
  uint32_t* arrive = nullptr;
  if (ext) {
    // fields are read only as far as the caller's struct reaches
    QMM_REQUIRE(ext->struct_size >= offsetof(qmm_gemm_ext, flags) + sizeof(ext->flags), QMM_ERR_INVALID_ARGUMENT,
                "%s: qmm_gemm_ext.struct_size (%zu) is too small", name, ext->struct_size);
    flags = ext->flags;
    if (ext->struct_size >= offsetof(qmm_gemm_ext, arrive_counter) + sizeof(ext->arrive_counter)) {
      signal = ext->done_signal;
      arrive = ext->arrive_counter;
    }
    QMM_REQUIRE((flags & ~(QMM_GEMM_INDEPENDENT | QMM_GEMM_STORE_MULTIMEM)) == 0, QMM_ERR_INVALID_ARGUMENT,
                "%s: unknown flag bits 0x%x", name, flags);
    QMM_REQUIRE((signal == nullptr) == (arrive == nullptr), QMM_ERR_INVALID_ARGUMENT,
                "%s: done_signal and arrive_counter go together", name);
    QMM_REQUIRE(aligned(signal, 4) && aligned(arrive, 4), QMM_ERR_INVALID_ARGUMENT, "%s: misaligned signal word", name);
  }
  if (M == 0 || N == 0) {
    QMM_REQUIRE(signal == nullptr, QMM_ERR_UNSUPPORTED, "%s: an empty result cannot signal", name);
    return QMM_OK;  // empty result
  }
  QMM_REQUIRE(x && w && scale && y, QMM_ERR_INVALID_ARGUMENT, "%s: null pointer", name);
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tma_ok = K > 0 && K % 8 == 0 && N % 16 == 0 && ldy % 2 == 0 && aligned(x, 16) &&
                      aligned(w, 16) && aligned(y, 4);
  if (tma_ok && M * N >= 128 * 128 && !force_simple())
    return w8a16_tcgen05(x, w, scale, y, M, N, K, ldy, flags, signal, arrive, s);
  QMM_REQUIRE(!(flags & QMM_GEMM_STORE_MULTIMEM) && signal == nullptr, QMM_ERR_UNSUPPORTED,
              "%s: multicast stores and completion signals need the tensor-core route "
              "(K %% 8 == 0, N %% 16 == 0, even ldy, 16-byte aligned x and w, M*N >= 16384)", name);
  QMM_REQUIRE(M <= 65535, QMM_ERR_UNSUPPORTED, "%s: unaligned shape with M > 65535", name);
  dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(M));
  simple::w8a16_kernel<<<grid, 128, 0, s>>>(x, w, scale, y, (int)M, (int)N, (int)K, (long long)ldy);
  QMM_CHECK_LAUNCH("w8a16_kernel(simple)");
  return QMM_OK;
}

int qmm_w8a16_perchannel(const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y,
                         int64_t M, int64_t N, int64_t K, int64_t ldy, void* stream) {
  return w8a16_entry("qmm_w8a16_perchannel", x, w, scale, y, M, N, K, ldy, nullptr, stream);
}

int qmm_w8a16_perchannel_ex(const uint16_t* x, const int8_t* w, const float* scale, uint16_t* y,
                            int64_t M, int64_t N, int64_t K, int64_t ldy, const qmm_gemm_ext* ext,
                            void* stream) {
  return w8a16_entry("qmm_w8a16_perchannel_ex", x, w, scale, y, M, N, K, ldy, ext, stream);
}

int qmm_wait_signals(const uint32_t* words, int count, uint32_t expected, uint64_t timeout_ns, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(words != nullptr && count >= 1 && count <= 4096 && aligned(words, 4), QMM_ERR_INVALID_ARGUMENT,
              "qmm_wait_signals: bad arguments");
  if (int st = read_device_status())
    return set_error(QMM_ERR_TIMEOUT, "a previous kernel gave up waiting (status word 0x%x)", st);
  if (timeout_ns == 0 || timeout_ns > 10000000000ull) timeout_ns = dev::kWaitLimitNs;
  simple::wait_words_kernel<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      words, count, expected, timeout_ns, device_status_word());
  QMM_CHECK_LAUNCH("wait_words_kernel");
  return QMM_OK;
}

int qmm_multicast_copy(const void* src, void* dst_multicast, size_t bytes, uint32_t* done_signal, uint32_t* arrive_counter,
                       int max_ctas, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(src && dst_multicast && done_signal && arrive_counter, QMM_ERR_INVALID_ARGUMENT,
              "qmm_multicast_copy: null pointer");
  QMM_REQUIRE(bytes % 16 == 0 && aligned(src, 16) && aligned(dst_multicast, 16) && aligned(done_signal, 4) &&
                  aligned(arrive_counter, 4),
              QMM_ERR_INVALID_ARGUMENT, "qmm_multicast_copy: bytes and pointers must be multiples of 16");
  QMM_REQUIRE(max_ctas >= 0 && max_ctas <= 1024, QMM_ERR_INVALID_ARGUMENT, "qmm_multicast_copy: bad max_ctas");
  if (bytes == 0) return QMM_OK;
  const size_t n16 = bytes / 16;
  int ctas = max_ctas == 0 ? 16 : max_ctas;
  const size_t need = (n16 + 511) / 512;
  if (static_cast<size_t>(ctas) > need) ctas = static_cast<int>(need);
  simple::multicast_copy_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst_multicast), n16, done_signal, arrive_counter);
  QMM_CHECK_LAUNCH("multicast_copy_kernel");
  return QMM_OK;
}

int qmm_peer_copy(const void* src, void* const* dst_peers, uint32_t* const* signal_peers, int n_peers, size_t bytes,
                  uint32_t* local_signal, uint32_t* arrive_counter, int max_ctas, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(src && dst_peers && signal_peers && local_signal && arrive_counter, QMM_ERR_INVALID_ARGUMENT,
              "qmm_peer_copy: null pointer");
  QMM_REQUIRE(n_peers >= 1 && n_peers <= QMM_MAX_PEERS, QMM_ERR_INVALID_ARGUMENT, "qmm_peer_copy: 1 to %d peers",
              QMM_MAX_PEERS);
  QMM_REQUIRE(bytes % 16 == 0 && aligned(src, 16) && aligned(local_signal, 4) && aligned(arrive_counter, 4),
              QMM_ERR_INVALID_ARGUMENT, "qmm_peer_copy: bytes and pointers must be multiples of 16");
  QMM_REQUIRE(max_ctas >= 0 && max_ctas <= 1024, QMM_ERR_INVALID_ARGUMENT, "qmm_peer_copy: bad max_ctas");
  simple::PeerList peers;
  peers.n = n_peers;
  for (int p = 0; p < n_peers; ++p) {
    QMM_REQUIRE(dst_peers[p] && signal_peers[p] && aligned(dst_peers[p], 16) && aligned(signal_peers[p], 4),
                QMM_ERR_INVALID_ARGUMENT, "qmm_peer_copy: peer %d: null or misaligned pointer", p);
    peers.dst[p] = static_cast<uint4*>(dst_peers[p]);
    peers.signal[p] = signal_peers[p];
  }
  if (bytes == 0) return QMM_OK;
  const size_t n16 = bytes / 16;
  int ctas = max_ctas == 0 ? 16 : max_ctas;
  const size_t need = (n16 + 511) / 512;
  if (static_cast<size_t>(ctas) > need) ctas = static_cast<int>(need);
  simple::peer_copy_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(src), peers, n16,
                                                                              local_signal, arrive_counter);
  QMM_CHECK_LAUNCH("peer_copy_kernel");
  return QMM_OK;
}

}  // extern "C"
