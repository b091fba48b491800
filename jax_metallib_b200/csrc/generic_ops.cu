// Standalone kernels for the small set of StableHLO ops that surround a quantized matmul.
//
// When the matcher fuses a dequantisation chain none of these run.  They exist so that a chain
// written in a way the matcher does not recognise — or the ops before and after a matmul — still
// executes on the GPU, op by op, with the semantics the reference implements for the same ops:
// convert (int -> float exact, float -> bf16 round-to-nearest-even: src/pjrt_plugin/ops/shape_ops.mm:662-829),
// multiply / subtract / add (floats computed in f32 and rounded to the result type, integers wrap:
// ops/binary_ops.mm:66-193), and / shift_right_logical (a shift >= the bit width gives 0:
// ops/bitwise_ops.mm:33-51,169-305), broadcast_in_dim / transpose / slice / concatenate
// (ops/shape_ops.mm:93-153,304-333,831-865,1265), splat constants (ops/tensor_creation_ops.mm:19-124)
// and a plain dot (f32 accumulation, one rounding; integer dots exact in int32 and wrapped to the
// result type: ops/binary_ops.mm:433-475,644-1245).  They are simple, HBM-bound, one launch per op.
#include "common.cuh"
#include "generic_ops.h"

namespace qmm {
namespace gen {

namespace {

__device__ __forceinline__ bool is_float_dt(int dt) { return dt == QMM_F32 || dt == QMM_F16 || dt == QMM_BF16; }

// element i of a tensor of type dt as float (floats) or as int (integers)
__device__ __forceinline__ float load_f(const void* p, int dt, long long i) {
  switch (dt) {
    case QMM_F32: return static_cast<const float*>(p)[i];
    case QMM_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case QMM_BF16: return dev::bf16_bits_to_float(static_cast<const uint16_t*>(p)[i]);
    default: return 0.f;
  }
}
__device__ __forceinline__ long long load_i(const void* p, int dt, long long i) {
  switch (dt) {
    case QMM_S8: return static_cast<const int8_t*>(p)[i];
    case QMM_U8: return static_cast<const uint8_t*>(p)[i];
    case QMM_S32: return static_cast<const int32_t*>(p)[i];
    case QMM_U32: return static_cast<const uint32_t*>(p)[i];
    case QMM_U4: return (static_cast<const uint8_t*>(p)[i >> 1] >> ((i & 1) * 4)) & 0xF;  // low nibble first
    default: return 0;
  }
}
__device__ __forceinline__ void store_f(void* p, int dt, long long i, float v) {
  switch (dt) {
    case QMM_F32: static_cast<float*>(p)[i] = v; break;
    case QMM_F16: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case QMM_BF16: static_cast<uint16_t*>(p)[i] = dev::float_to_bf16_bits(v); break;
    default: break;
  }
}
__device__ __forceinline__ void store_i(void* p, int dt, long long i, long long v) {  // wraps to the type's width
  switch (dt) {
    case QMM_S8: static_cast<int8_t*>(p)[i] = static_cast<int8_t>(v); break;
    case QMM_U8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v); break;
    case QMM_S32: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    case QMM_U32: static_cast<uint32_t*>(p)[i] = static_cast<uint32_t>(v); break;
    default: break;
  }
}
__device__ __forceinline__ int bit_width(int dt) {
  return (dt == QMM_S8 || dt == QMM_U8) ? 8 : (dt == QMM_U4 ? 4 : 32);
}

__global__ void convert_kernel(const void* in, int in_dt, void* out, int out_dt, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (is_float_dt(out_dt)) {
      const float v = is_float_dt(in_dt) ? load_f(in, in_dt, i) : static_cast<float>(load_i(in, in_dt, i));
      store_f(out, out_dt, i, v);
    } else {
      store_i(out, out_dt, i, load_i(in, in_dt, i));  // integer -> integer: wraps to the result width
    }
  }
}

__global__ void binary_kernel(int op, const void* a, const void* b, void* out, int dt, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (is_float_dt(dt)) {
      const float x = load_f(a, dt, i), y = load_f(b, dt, i);
      const float r = op == kMul ? x * y : (op == kSub ? x - y : x + y);
      store_f(out, dt, i, r);
    } else {
      const long long x = load_i(a, dt, i), y = load_i(b, dt, i);
      long long r = 0;
      switch (op) {
        case kMul: r = x * y; break;
        case kSub: r = x - y; break;
        case kAdd: r = x + y; break;
        case kAnd: r = x & y; break;
        case kShrLogical: {
          const int w = bit_width(dt);
          const unsigned long long ux = static_cast<unsigned long long>(x) & ((w == 32) ? 0xFFFFFFFFull : ((1ull << w) - 1));
          const unsigned long long sh = static_cast<unsigned long long>(y) & ((w == 32) ? 0xFFFFFFFFull : ((1ull << w) - 1));
          r = (sh >= static_cast<unsigned long long>(w)) ? 0 : static_cast<long long>(ux >> sh);
          break;
        }
      }
      store_i(out, dt, i, r);
    }
  }
}

struct Shape4 {
  long long d[kMaxRank];
};

// out[o] = in[index built from the out coordinates through `src_of`]: broadcast_in_dim (src_of[k] = the
// out dimension that in dimension k reads, size-1 in dimensions read coordinate 0), transpose
// (src_of[k] = out dimension holding in dimension k) and slice (start/stride per dimension).
__global__ void gather_kernel(const uint8_t* in, uint8_t* out, int esz, int in_rank, Shape4 in_dims, int out_rank,
                              Shape4 out_dims, Shape4 src_of, Shape4 start, Shape4 stride, long long n) {
  for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < n;
       o += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long coord[kMaxRank];
    long long rem = o;
    for (int k = out_rank - 1; k >= 0; --k) {
      coord[k] = rem % out_dims.d[k];
      rem /= out_dims.d[k];
    }
    long long idx = 0;
    for (int k = 0; k < in_rank; ++k) {
      long long c = in_dims.d[k] == 1 ? 0 : coord[src_of.d[k]];
      c = start.d[k] + c * stride.d[k];
      idx = idx * in_dims.d[k] + c;
    }
    for (int b = 0; b < esz; ++b) out[o * esz + b] = in[idx * esz + b];
  }
}

// out[.., offset + j, ..] = in[.., j, ..] along one dimension: `outer` x `in_len` x `inner` elements
__global__ void concat_part_kernel(const uint8_t* in, uint8_t* out, int esz, long long outer, long long in_len,
                                   long long out_len, long long offset, long long inner) {
  const long long n = outer * in_len * inner;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long in_i = i % inner, j = (i / inner) % in_len, o = i / (inner * in_len);
    const long long dst = (o * out_len + offset + j) * inner + in_i;
    for (int b = 0; b < esz; ++b) out[dst * esz + b] = in[i * esz + b];
  }
}

__global__ void fill_kernel(void* out, int dt, double fv, long long iv, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (is_float_dt(dt)) store_f(out, dt, i, static_cast<float>(fv));
    else store_i(out, dt, i, iv);
  }
}

// out[m, n] = sum_k a[m, k] * b[k, n] (or b[n, k] when b_transposed); 16 x 16 tiles through shared memory
__global__ void dot_kernel(const void* a, const void* b, void* out, int in_dt, int out_dt, int M, int N, int K,
                           int b_transposed) {
  __shared__ float sa[16][17], sb[16][17];
  __shared__ int ia[16][17], ib[16][17];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int m = blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx;
  const bool fl = is_float_dt(in_dt);
  float facc = 0.f;
  int iacc = 0;  // wraps mod 2^32 like the reference's int32 accumulator
  for (int k0 = 0; k0 < K; k0 += 16) {
    const int ka = k0 + tx, kb = k0 + ty;
    const long long ai = static_cast<long long>(m) * K + ka;
    const long long bi = b_transposed ? static_cast<long long>(n) * K + kb : static_cast<long long>(kb) * N + n;
    if (fl) {
      sa[ty][tx] = (m < M && ka < K) ? load_f(a, in_dt, ai) : 0.f;
      sb[ty][tx] = (n < N && kb < K) ? load_f(b, in_dt, bi) : 0.f;
    } else {
      ia[ty][tx] = (m < M && ka < K) ? static_cast<int>(load_i(a, in_dt, ai)) : 0;
      ib[ty][tx] = (n < N && kb < K) ? static_cast<int>(load_i(b, in_dt, bi)) : 0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (fl) facc = fmaf(sa[ty][k], sb[k][tx], facc);
      else iacc = static_cast<int>(static_cast<unsigned>(iacc) + static_cast<unsigned>(ia[ty][k] * ib[k][tx]));
    }
    __syncthreads();
  }
  if (m < M && n < N) {
    const long long o = static_cast<long long>(m) * N + n;
    if (is_float_dt(out_dt)) store_f(out, out_dt, o, fl ? facc : static_cast<float>(iacc));
    else store_i(out, out_dt, o, iacc);
  }
}

unsigned grid_for(long long n) {
  long long g = (n + 255) / 256;
  const long long cap = 148ll * 16;
  return static_cast<unsigned>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

size_t dtype_bits(int dt) {
  switch (dt) {
    case QMM_F32: case QMM_S32: case QMM_U32: return 32;
    case QMM_F16: case QMM_BF16: return 16;
    case QMM_S8: case QMM_U8: return 8;
    case QMM_U4: return 4;
    default: return 0;
  }
}

int convert(const void* in, int in_dt, void* out, int out_dt, long long n, cudaStream_t s) {
  QMM_REQUIRE(out_dt != QMM_U4, QMM_ERR_UNSUPPORTED, "convert to a 4-bit type is not supported");
  QMM_REQUIRE(!(in_dt == QMM_F32 || in_dt == QMM_F16 || in_dt == QMM_BF16) ||
                  (out_dt == QMM_F32 || out_dt == QMM_F16 || out_dt == QMM_BF16),
              QMM_ERR_UNSUPPORTED, "convert from a float to an integer type is not supported");
  if (n == 0) return QMM_OK;
  convert_kernel<<<grid_for(n), 256, 0, s>>>(in, in_dt, out, out_dt, n);
  QMM_CHECK_LAUNCH("convert_kernel");
  return QMM_OK;
}

int binary(int op, const void* a, const void* b, void* out, int dt, long long n, cudaStream_t s) {
  const bool fl = dt == QMM_F32 || dt == QMM_F16 || dt == QMM_BF16;
  QMM_REQUIRE(dt != QMM_U4, QMM_ERR_UNSUPPORTED, "arithmetic on 4-bit tensors is not supported");
  QMM_REQUIRE(!(fl && (op == kAnd || op == kShrLogical)), QMM_ERR_UNSUPPORTED, "bitwise op on a float tensor");
  if (n == 0) return QMM_OK;
  binary_kernel<<<grid_for(n), 256, 0, s>>>(op, a, b, out, dt, n);
  QMM_CHECK_LAUNCH("binary_kernel");
  return QMM_OK;
}

int gather(const void* in, void* out, int dt, const long long* in_dims, int in_rank, const long long* out_dims,
           int out_rank, const long long* src_of, const long long* start, const long long* stride, cudaStream_t s) {
  QMM_REQUIRE(in_rank <= kMaxRank && out_rank <= kMaxRank && in_rank >= 0 && out_rank >= 0, QMM_ERR_UNSUPPORTED,
              "tensors of rank > %d are not supported", kMaxRank);
  QMM_REQUIRE(dtype_bits(dt) >= 8, QMM_ERR_UNSUPPORTED, "shape ops on 4-bit tensors are not supported");
  Shape4 id = {}, od = {}, so = {}, st = {}, sr = {};
  long long n = 1;
  for (int k = 0; k < out_rank; ++k) {
    od.d[k] = out_dims[k];
    n *= out_dims[k];
  }
  for (int k = 0; k < in_rank; ++k) {
    id.d[k] = in_dims[k];
    so.d[k] = src_of[k];
    st.d[k] = start ? start[k] : 0;
    sr.d[k] = stride ? stride[k] : 1;
  }
  if (n == 0) return QMM_OK;
  gather_kernel<<<grid_for(n), 256, 0, s>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out),
                                           static_cast<int>(dtype_bits(dt) / 8), in_rank, id, out_rank, od, so, st, sr, n);
  QMM_CHECK_LAUNCH("gather_kernel");
  return QMM_OK;
}

int concat_part(const void* in, void* out, int dt, long long outer, long long in_len, long long out_len,
                long long offset, long long inner, cudaStream_t s) {
  QMM_REQUIRE(dtype_bits(dt) >= 8, QMM_ERR_UNSUPPORTED, "shape ops on 4-bit tensors are not supported");
  const long long n = outer * in_len * inner;
  if (n == 0) return QMM_OK;
  concat_part_kernel<<<grid_for(n), 256, 0, s>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out),
                                                static_cast<int>(dtype_bits(dt) / 8), outer, in_len, out_len, offset, inner);
  QMM_CHECK_LAUNCH("concat_part_kernel");
  return QMM_OK;
}

int fill(void* out, int dt, double fv, long long iv, long long n, cudaStream_t s) {
  QMM_REQUIRE(dt != QMM_U4, QMM_ERR_UNSUPPORTED, "4-bit constants are not supported");
  if (n == 0) return QMM_OK;
  fill_kernel<<<grid_for(n), 256, 0, s>>>(out, dt, fv, iv, n);
  QMM_CHECK_LAUNCH("fill_kernel");
  return QMM_OK;
}

int dot(const void* a, const void* b, void* out, int in_dt, int out_dt, long long M, long long N, long long K,
        int b_transposed, cudaStream_t s) {
  QMM_REQUIRE(in_dt != QMM_U4 && out_dt != QMM_U4, QMM_ERR_UNSUPPORTED, "dot on 4-bit tensors is not supported");
  QMM_REQUIRE(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), QMM_ERR_UNSUPPORTED, "dot too large");
  const bool fl = in_dt == QMM_F32 || in_dt == QMM_F16 || in_dt == QMM_BF16;
  const bool flo = out_dt == QMM_F32 || out_dt == QMM_F16 || out_dt == QMM_BF16;
  QMM_REQUIRE(!fl || flo, QMM_ERR_UNSUPPORTED, "a float dot with an integer result is not supported");
  if (M == 0 || N == 0) return QMM_OK;
  QMM_REQUIRE((M + 15) / 16 <= 65535, QMM_ERR_UNSUPPORTED, "dot with M > 1048560 is not supported");
  dim3 grid(static_cast<unsigned>((N + 15) / 16), static_cast<unsigned>((M + 15) / 16));
  dot_kernel<<<grid, dim3(16, 16), 0, s>>>(a, b, out, in_dt, out_dt, (int)M, (int)N, (int)K, b_transposed);
  QMM_CHECK_LAUNCH("dot_kernel");
  return QMM_OK;
}

}  // namespace gen
}  // namespace qmm
