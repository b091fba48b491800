// Host entry points of the standalone op kernels (generic_ops.cu), used by the StableHLO planner
// for ops it does not fuse into a matmul.  All take device pointers and a stream.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace qmm {
namespace gen {

constexpr int kMaxRank = 4;
enum BinaryOp { kMul = 0, kSub = 1, kAdd = 2, kAnd = 3, kShrLogical = 4 };

size_t dtype_bits(int dtype);  // of a qmm_dtype; 0 for an unknown tag

int convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream);
int binary(int op, const void* a, const void* b, void* out, int dtype, long long n, cudaStream_t stream);
// out[coords] = in[...]: input dimension k reads output dimension src_of[k] (coordinate 0 when the
// input dimension has size 1), scaled by stride[k] and offset by start[k] (both may be null).
int gather(const void* in, void* out, int dtype, const long long* in_dims, int in_rank, const long long* out_dims,
           int out_rank, const long long* src_of, const long long* start, const long long* stride,
           cudaStream_t stream);
// One operand of a concatenate: [outer, in_len, inner] into [outer, out_len, inner] at `offset`.
int concat_part(const void* in, void* out, int dtype, long long outer, long long in_len, long long out_len,
                long long offset, long long inner, cudaStream_t stream);
int fill(void* out, int dtype, double float_value, long long int_value, long long n, cudaStream_t stream);
// out[M, N] = a[M, K] . b[K, N] (b[N, K] when b_transposed): f32 accumulate for floats, wrapping
// int32 accumulate for integers, one conversion to out_dtype.
int dot(const void* a, const void* b, void* out, int in_dtype, int out_dtype, long long M, long long N, long long K,
        int b_transposed, cudaStream_t stream);

}  // namespace gen
}  // namespace qmm
