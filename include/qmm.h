/*
 * qmm.h — C ABI of the B200 quantized-matmul kernel library (libqmm.so).
 *
 * This is the drop-in boundary for the quantized-matmul hot path of
 * erfanzar/jax-metallib.  Every entry point takes plain device pointers, sizes
 * and a CUDA stream (passed as void*, i.e. a cudaStream_t); nothing in the
 * signatures depends on PyTorch, JAX or C++ types.  All tensors are dense and
 * row-major unless a leading dimension is given.  Kernel entry points are
 * asynchronous on the given stream and allocate no device memory: scratch,
 * where a kernel needs it, is passed in by the caller (see the
 * *_workspace_bytes queries) or, for qmm_w4a16_g128_static_scratch, is a fixed
 * array inside the library.  The runtime objects of qmm_rt.h (buffers, events,
 * executables) do allocate; they are a separate layer on top of these calls.
 *
 * Each function names the interface of the reference it stands in for
 * (paths relative to the reference project root).
 *
 * Return value: 0 (QMM_OK) or a qmm_status error code; a human-readable
 * message for the calling thread's last failure is available through
 * qmm_last_error().  No function throws or aborts, and there is no CPU
 * fallback: an unsupported shape or dtype is an error, as a missing op is in
 * the reference's compile step (src/pjrt_plugin/api/pjrt_client.cc:211-220).
 */
#ifndef QMM_H_
#define QMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QMM_API
#else
#define QMM_API __attribute__((visibility("default")))
#endif

typedef enum qmm_status {
  QMM_OK = 0,
  QMM_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad size, misaligned pointer */
  QMM_ERR_UNSUPPORTED = 2,      /* shape / dtype / mode outside what the kernels cover */
  QMM_ERR_CUDA = 3,             /* a CUDA runtime or driver call failed */
  QMM_ERR_WORKSPACE = 4,        /* workspace missing or too small */
  QMM_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up */
  QMM_ERR_PARSE = 6             /* StableHLO text could not be read or matched */
} qmm_status;

/* Element type tags used by the entry points that take void* tensors. */
typedef enum qmm_dtype {
  QMM_F32 = 0,
  QMM_F16 = 1,
  QMM_BF16 = 2,
  QMM_S8 = 3,
  QMM_U8 = 4,
  QMM_S32 = 5,
  QMM_U4 = 6, /* two values per byte, low nibble first */
  QMM_U32 = 7
} qmm_dtype;

/* MX microscaling modes of the operator API
 * (src/jax_plugins/silicon/quantized.py:39-43). */
typedef enum qmm_mx_mode { QMM_MXFP4 = 0, QMM_MXFP8 = 1, QMM_NVFP4 = 2 } qmm_mx_mode;

QMM_API const char* qmm_version(void);
QMM_API const char* qmm_status_name(int status);
/* Copies the calling thread's last error message (NUL-terminated, truncated to
 * cap) and returns its full length.  Mirrors the reference's error-as-value
 * convention (src/pjrt_plugin/api/pjrt_memory.cc:22-57). */
QMM_API size_t qmm_last_error(char* buf, size_t cap);

/* Device-side waits (mbarrier / flag polls inside the kernels) are bounded: a
 * kernel that gives up writes QMM_ERR_TIMEOUT plus a site tag into a
 * host-visible status word and returns normally.  qmm_device_status() reads
 * that word without synchronising (0 = healthy); entry points refuse further
 * launches while it is set; qmm_clear_device_status() resets it.  The
 * reference's counterpart is the bounded caller wait that returns
 * DEADLINE_EXCEEDED (src/pjrt_plugin/core/completion_event.h:62-83,
 * src/pjrt_plugin/api/pjrt_event.cc:46-59). */
QMM_API int qmm_device_status(void);
/* Host-only self-check of the library's internal bookkeeping (per-device
 * "configured once" masks, cached environment switches).  Needs no GPU.
 * Returns 0 when every check passes.  No reference counterpart. */
QMM_API int qmm_selftest_host(void);
QMM_API void qmm_clear_device_status(void);

/* Upper bound on the CTAs of the persistent tcgen05 GEMMs (qmm_w8a16_perchannel,
 * qmm_i8i8_i32); 0 = one per SM (the default).  Those kernels keep one CTA per
 * SM resident for the whole launch, so a communication kernel that should run
 * next to them (an NCCL all-gather of the previous output on a second stream)
 * finds no SM unless some are left free; a tensor-parallel caller sets the
 * limit to the SM count minus the CTAs its collective uses.  Process-wide.
 * No reference counterpart (the reference runs one device). */
QMM_API int qmm_set_cta_limit(int max_ctas);

/* ---------------------------------------------------------------------------
 * Weight-only int8, per-output-channel scale, f32 activations.
 *   y[M,N] = x[M,K] @ (float(w[K,N]) * scale[N])
 * Replaces the un-fused chain HandleConvert -> HandleBroadcastInDim ->
 * HandleMultiply -> HandleDotGeneral
 * (src/pjrt_plugin/ops/shape_ops.mm:793-829, :93-153;
 *  src/pjrt_plugin/ops/binary_ops.mm:165-193, :1006-1019).
 * Exact f32 FMA arithmetic; the scale is applied once per output element. */
QMM_API int qmm_w8a32_perchannel(const float* x, const int8_t* w, const float* scale, float* y,
                                 int64_t M, int64_t N, int64_t K, void* stream);

/* ---------------------------------------------------------------------------
 * Weight-only int8, per-output-channel scale, bf16 activations, bf16 output.
 *   y[M, ldy] (columns 0..N-1) = bf16( (x[M,K] @ float(w[K,N])) * scale[N] )
 * Same chain as above with a bf16 lhs (src/pjrt_plugin/ops/binary_ops.mm:740-805:
 * bf16 operands, f32 accumulation, one rounding to the declared result type).
 * ldy is the row stride of y in elements (>= N), so that a rank holding a
 * column shard can write straight into its slice of the gathered output.
 * tcgen05 (kind::f16) GEMM with the int8->bf16 conversion done in shared
 * memory.  The tensor-core route needs K % 8 == 0, N % 16 == 0, an even ldy
 * and 16-byte aligned x and w (what TMA can address); any other shape runs on
 * a plain CUDA-core kernel. */
QMM_API int qmm_w8a16_perchannel(const uint16_t* x_bf16, const int8_t* w, const float* scale,
                                 uint16_t* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldy,
                                 void* stream);
/* The same matmul with launch options (a struct led by its own size, so that
 * fields can be added; only the fields inside struct_size are read).
 *
 * QMM_GEMM_INDEPENDENT: the caller states that no launch of this entry point
 *   queued earlier on the stream, back to and including the last one made
 *   without this flag, writes x, w or scale or touches y.  The launch then does
 *   not order itself behind those launches, and its first tiles run on the SMs
 *   that its predecessor's last, partly filled round leaves idle.  A launch
 *   without the flag waits for everything ahead of it on the stream before it
 *   touches memory, and holds back its successors until it has done so; so a
 *   flagged launch never overlaps anything older than the last unflagged one.
 *   (Kernels of other entry points between two launches order them fully,
 *   except the decode operators, which start early behind their predecessor:
 *   do not put a flagged launch directly behind those.)
 * QMM_GEMM_STORE_MULTIMEM: y is a multicast (NVSwitch multimem) address: every
 *   store of the epilogue lands at the same offset of the buffer of every GPU
 *   bound to the multicast object, this one included.  This is the all-gather
 *   of a column-sharded linear (stablehlo.all_gather over one replica group;
 *   the reference's handler is src/pjrt_plugin/ops/collective_ops.mm:88-229,
 *   an identity on its single device) done by the GEMM's own stores: rank r
 *   passes the multicast address of block r of the gathered [P, M, N/P] buffer.
 * done_signal / arrive_counter (both or neither): when the launch's stores are
 *   complete, done_signal (a multicast address under QMM_GEMM_STORE_MULTIMEM)
 *   is incremented by 1 with release semantics at system scope; a reader that
 *   observes the count with an acquire load (qmm_wait_signals) may read the
 *   output.  arrive_counter is a local uint32, zero before its first use and
 *   left zero, on which the launch's CTAs count themselves. */
#define QMM_GEMM_INDEPENDENT 1u
#define QMM_GEMM_STORE_MULTIMEM 2u
typedef struct qmm_gemm_ext {
  size_t struct_size; /* sizeof(qmm_gemm_ext) as the caller knows it */
  uint32_t flags;
  uint32_t* done_signal;
  uint32_t* arrive_counter;
} qmm_gemm_ext;
QMM_API int qmm_w8a16_perchannel_ex(const uint16_t* x_bf16, const int8_t* w, const float* scale,
                                    uint16_t* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldy,
                                    const qmm_gemm_ext* ext, void* stream);
/* Queues a kernel that waits until words[i] >= expected for all i < count
 * (the done_signal words of the ranks of a sharded linear), for at most
 * timeout_ns (0 = the library's 2 s default).  A wait that runs out records
 * QMM_ERR_TIMEOUT in the device status word and the kernel returns, so the
 * context stays usable; the reference's counterpart is the bounded event wait
 * (src/pjrt_plugin/core/completion_event.h:62-83).  The words must be written
 * by other GPUs (or be set already), never by a kernel queued on this GPU after
 * the wait. */
QMM_API int qmm_wait_signals(const uint32_t* words, int count, uint32_t expected, uint64_t timeout_ns,
                             void* stream);
/* The all-gather of a finished block as a kernel of its own: copies `bytes`
 * (a multiple of 16; both pointers 16-byte aligned) from local memory to a
 * multicast (NVSwitch multimem) address, 16 bytes per thread and fully
 * coalesced, so that every GPU bound to the multicast object receives the
 * block at that offset; then adds 1 to done_signal (a multicast address) with
 * release semantics at system scope, as qmm_w8a16_perchannel_ex does.
 * arrive_counter is a local uint32, zero before its first use and left zero.
 * max_ctas bounds the grid (0 = 16): the copy is meant to run beside a GEMM
 * that leaves those SMs free (qmm_set_cta_limit).  Replaces the same
 * reference handler as QMM_GEMM_STORE_MULTIMEM
 * (src/pjrt_plugin/ops/collective_ops.mm:88-229) where link efficiency
 * matters more than the SMs the copy occupies: the GEMM epilogue's stores
 * reach the switch as 64-byte runs, these as 512-byte runs. */
QMM_API int qmm_multicast_copy(const void* src, void* dst_multicast, size_t bytes, uint32_t* done_signal,
                               uint32_t* arrive_counter, int max_ctas, void* stream);
/* The same all-gather step with plain peer stores instead of a multicast
 * address: every 16 bytes read from src are stored to dst_peers[0..n_peers-1]
 * (the block's address in each peer GPU's buffer; peer-mapped pointers, at most
 * QMM_MAX_PEERS), then signal_peers[i] (the word of this rank in peer i's
 * buffer) and local_signal are each incremented by 1 with release semantics at
 * system scope.  A multicast store also delivers the block to the sender's own
 * buffer, 1/P of the arriving bytes; when the links are the bound (P = 8 on
 * NVLink 5: 55 GB of gathered outputs per step of the headline workload
 * against 66 ms of GEMM) leaving that out is worth more than the P-1 stores
 * per load cost.  max_ctas bounds the grid (0 = 16). */
#define QMM_MAX_PEERS 15
QMM_API int qmm_peer_copy(const void* src, void* const* dst_peers, uint32_t* const* signal_peers, int n_peers,
                          size_t bytes, uint32_t* local_signal, uint32_t* arrive_counter, int max_ctas, void* stream);

/* ---------------------------------------------------------------------------
 * int8 x int8 -> int32 dot with optional fused f32 rescale.
 *   acc[M,N]  = a[M,K] . b[K,N]            (exact, int32)          if acc != NULL
 *   out[M,N]  = float(acc) * row_scale[M] * col_scale[N]           if out != NULL
 * Replaces IntegerMatMul (src/pjrt_plugin/ops/binary_ops.mm:433-475), which
 * the reference emulates as an [M,K,N] broadcast product reduced over K, and
 * the convert/multiply/multiply that follow it (ops/shape_ops.mm:793-829,
 * ops/binary_ops.mm:165-193).  The multiplies happen in that order, each
 * rounded to f32.  a_unsigned / b_unsigned select uint8 operands
 * (tests/test_dot_preferred_dtype.py:61). */
QMM_API int qmm_i8i8_i32(const void* a, const void* b, int32_t* acc, const float* row_scale,
                         const float* col_scale, float* out, int64_t M, int64_t N, int64_t K,
                         int a_unsigned, int b_unsigned, void* stream);

/* ---------------------------------------------------------------------------
 * int4 asymmetric group-wise weight-only matmul, decode and prefill sizes.
 *   w[k,n] = (q[k,n] - z[k/group, n]) * s[k/group, n]
 *   y[M,N] = bf16( x[M,K] @ w[K,N] )
 * wq is uint8 [K/2, N]: byte [kk, n] holds q[2kk, n] in its low nibble and
 * q[2kk+1, n] in its high nibble (the reference's low-nibble-first packing,
 * src/jax_plugins/silicon/quantized.py:189-191,264).  scales are bf16
 * [K/group, N]; zeros are [K/group, N] one per byte (zeros_packed = 0) or
 * [K/group, N/2] two per byte, low nibble = even n (zeros_packed = 1).
 * Replaces and(…,15) / shift_right_logical(…,4) / convert / subtract /
 * multiply / reshape / dot_general
 * (src/pjrt_plugin/ops/bitwise_ops.mm:33-51,169-305; ops/shape_ops.mm:793-829;
 *  ops/binary_ops.mm:66-193, :644-1245).
 * Zero points are 4-bit values (0..15) in either form.
 * Requires group == 128, K % 128 == 0, N % 128 == 0, M >= 1.
 * M <= 32 runs the HBM-bound decode kernel (weights read once, split-K over
 * all SMs); larger M runs a tcgen05 GEMM whose converter warps dequantise the
 * nibbles in shared memory: bf16((q - z) * s) per weight, which is what the
 * StableHLO chain computes in bf16, f32 accumulation, one rounding of the
 * result.  That route needs no workspace (qmm_w4a16_g128_workspace_bytes
 * returns 0 for M > 32 and workspace may be NULL) and ignores flags.
 * workspace (M <= 32): qmm_w4a16_g128_workspace_bytes(M, N, K) bytes, 256-byte
 * aligned, zero-filled before its first use; the kernel leaves it zero-filled,
 * so back-to-back calls on one stream may share it.
 * flags: 0, or QMM_W4_STATIC_WEIGHTS when wq, scales and zeros are not written
 * by any work queued earlier on the stream (the usual case for model weights).
 * The kernel is launched with programmatic stream serialization: its blocks
 * may start while the previous kernel on the stream drains.  x, y and the
 * workspace are only touched once that kernel has finished; with
 * QMM_W4_STATIC_WEIGHTS the first weight tiles are fetched before that point,
 * which hides the launch gap in a decode loop. */
#define QMM_W4_STATIC_WEIGHTS 1u
QMM_API size_t qmm_w4a16_g128_workspace_bytes(int64_t M, int64_t N, int64_t K);
QMM_API int qmm_w4a16_g128(const uint16_t* x_bf16, const uint8_t* wq, const uint16_t* scales_bf16,
                           const uint8_t* zeros, int zeros_packed, uint16_t* y_bf16, int64_t M,
                           int64_t N, int64_t K, int64_t group, void* workspace,
                           size_t workspace_bytes, unsigned flags, void* stream);

/* ---------------------------------------------------------------------------
 * The same matmul for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference; it exists for hosts
 * of this library that must not (or cannot) call cudaMalloc around a matmul:
 * an executable running under a runtime that already owns nearly all of HBM
 * (a PJRT/XLA client preallocates its pool, so a later cudaMalloc can simply
 * fail), and decode loops in which an allocation or free would synchronise
 * the whole device in the middle of a token.  Such a caller has nowhere to
 * get the split-K workspace of qmm_w4a16_g128 from, so this variant brings its
 * own: a fixed array of QMM_STATIC_SCRATCH_BYTES inside the library's device
 * image (each GPU that loads the library holds it until the process exits).
 *
 * Arguments and result are those of qmm_w4a16_g128 without the workspace.
 * The call allocates nothing and frees nothing.  Limits and rules:
 *  - shapes whose scratch need (qmm_w4a16_g128_workspace_bytes) exceeds
 *    QMM_STATIC_SCRATCH_BYTES are refused with QMM_ERR_WORKSPACE — 8 MiB covers
 *    M <= 16 at 4096 x 14336 (6.4 MB) and at 14336 x 4096;
 *  - the first call on each device resolves the array's device address; make
 *    that call before starting any stream capture;
 *  - the array is shared by every call on the device and keeps what the last
 *    call wrote; the part that must start at zero is cleared on the stream by
 *    each call, but two calls that may run at the same time on one GPU race
 *    on it — keep them on one stream or order them yourself;
 *  - a device-side wait that gives up is recorded in the status word of
 *    qmm_device_status() only if that word exists when the kernel is launched;
 *    creating it allocates pinned host memory, which this call will not do, so
 *    call qmm_device_status() once during start-up if you want such timeouts
 *    reported (and later launches refused) here as well. */
#define QMM_STATIC_SCRATCH_BYTES (8u << 20)
QMM_API int qmm_w4a16_g128_static_scratch(const uint16_t* x_bf16, const uint8_t* wq,
                                          const uint16_t* scales_bf16, const uint8_t* zeros,
                                          int zeros_packed, uint16_t* y_bf16, int64_t M, int64_t N,
                                          int64_t K, int64_t group, void* stream);

/* ---------------------------------------------------------------------------
 * Operator-API formats (weights stored transposed, [N, ...], K contiguous).
 *
 * qmm_affine_matmul replaces affine_quantized_matmul / _affine_matmul_gpu and
 * the affine_qgemm_{4,8}bit_{f32,f16} kernels
 * (src/jax_plugins/silicon/quantized.py:772-957, :1077-1152):
 *   y[M,N] = dtype( sum_k float(x[m,k]) * (scales[n,k/gs] * q[n,k] + biases[n,k/gs]) )
 * bits = 4: w_packed is uint32 [N, K/8], value j of a word at bits 4j;
 * bits = 8: w_packed is uint8 [N, K].  dtype = QMM_F32 or QMM_F16 (x and y).
 *
 * qmm_mx_matmul replaces quantized_matmul / _quantized_matmul_gpu and the
 * mx_qgemm_{mxfp4,mxfp8,nvfp4}_{f32,f16} kernels (quantized.py:528-753,
 * :995-1074): E2M1 / E4M3 elements, E8M0 (group 32) or E4M3 (group 16) scales,
 * NaN codes (E4M3 0x7F/0xFF, E8M0 0xFF) propagate.
 *
 * Both choose a kernel by shape.  With f16 activations and M <= 16 (decode) the
 * packed codes go to the tensor cores from per-warp TMA rings when x, w_packed,
 * scales (and biases) are 16-byte aligned, N is a multiple of 16 and, affine:
 * group_size is 64 / 128 / 256 (4-bit) or 32 / 64 / 128 (8-bit) with a multiple
 * of 4 groups per row; MX: K is a multiple of 512 (mxfp4, mxfp8) or 256
 * (nvfp4).  Other shapes, M > 16 and f32 activations run on CUDA-core kernels
 * with the same arithmetic (scale * q + bias or scale * element in f32, f32
 * accumulation, one cast).  The tensor-core kernels apply the scale per group
 * instead of per weight: same result up to f32 rounding of the sums. */
QMM_API int qmm_affine_matmul(const void* x, const void* w_packed, const float* scales,
                              const float* biases, void* y, int64_t M, int64_t N, int64_t K,
                              int bits, int64_t group_size, int dtype, void* stream);
QMM_API int qmm_mx_matmul(const void* x, const uint8_t* w_packed, const uint8_t* scales, void* y,
                          int64_t M, int64_t N, int64_t K, int mode, int dtype, void* stream);

/* ---------------------------------------------------------------------------
 * The other operators of a Llama-shaped int4 decode step (bf16 activations).
 * In the reference these are MPSGraph nodes or its native row kernels
 * (take-rows fusion src/pjrt_plugin/core/mps_executable.mm:1149-1160,
 * row reductions and softmax runtime/metal_kernels.mm:769-1170,1422-1950,
 * elementwise ops ops/unary_ops.mm, ops/binary_ops.mm:66-193, batched dots
 * ops/binary_ops.mm:1193-1212); here each is one CUDA launch.
 *
 * qmm_take_rows_bf16: out[b,:] = table[ids[b],:]; negative ids count from the
 *   end, out-of-range ids give rows of `fill_bits` (README.md:200-202).
 * qmm_add_rmsnorm_bf16: h = x + residual (residual may be NULL), rounded to
 *   bf16 and stored to sum_out if given; norm_out =
 *   bf16(bf16(h * rsqrt(mean(h^2) + eps)) * weight), statistics in f32.
 * qmm_rope_bf16: rotary embedding in place on q [B,Hq,hd] and k [B,Hkv,hd],
 *   pairs (i, i + hd/2), angle = position * theta^(-2i/hd); batch rows of q / k
 *   are q_ld / k_ld elements apart (slices of a fused q|k|v projection output).
 * qmm_silu_mul_bf16: out = bf16(bf16(silu(gate)) * up); gate/up rows are ld_in
 *   elements apart (so they may be the two halves of one buffer).
 * qmm_attention_decode_bf16: grouped-query attention of one new token per
 *   sequence over a read-only cache [B,Hkv,L,128] plus the new key/value row
 *   [B,Hkv,128]; batch rows of q are q_ld elements apart, those of knew / vnew
 *   new_ld; scores and P.V on the tensor cores (bf16 operands, f32 accumulate),
 *   softmax in f32; two launches (per-split partials, merge).  flags:
 *   QMM_ATTN_STATIC_CACHE states that no kernel still in flight on the stream
 *   writes the cache (a step that returns the new rows instead of appending
 *   them), so that the cache may be fetched before those kernels finish.
 * qmm_bf16_matmul_small_m: y[M,N] = bf16(x[M,K] @ w[K,N]), bf16 operands, f32
 *   accumulate, M <= 16 (the unquantized lm_head of the decode step).
 * All of these start early behind the previous kernel of the stream
 * (programmatic stream serialization) and wait for it before touching data. */
#define QMM_ATTN_STATIC_CACHE 1u
QMM_API int qmm_take_rows_bf16(const uint16_t* table, const int32_t* ids, uint16_t* out, int64_t V,
                               int64_t D, int64_t B, uint16_t fill_bits, void* stream);
QMM_API int qmm_add_rmsnorm_bf16(const uint16_t* x, const uint16_t* residual, const uint16_t* weight,
                                 uint16_t* sum_out, uint16_t* norm_out, int64_t B, int64_t D,
                                 float eps, void* stream);
QMM_API int qmm_rope_bf16(uint16_t* q, uint16_t* k, const int32_t* positions, int64_t B, int64_t Hq,
                          int64_t Hkv, int64_t head_dim, float theta, int64_t q_ld, int64_t k_ld,
                          void* stream);
QMM_API int qmm_silu_mul_bf16(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t B,
                              int64_t F, int64_t ld_in, void* stream);
QMM_API size_t qmm_attention_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t L);
QMM_API int qmm_attention_decode_bf16(const uint16_t* q, const uint16_t* kcache,
                                      const uint16_t* vcache, const uint16_t* knew,
                                      const uint16_t* vnew, uint16_t* out, int64_t B, int64_t Hq,
                                      int64_t Hkv, int64_t L, int64_t head_dim, float scale,
                                      int64_t q_ld, int64_t new_ld, void* workspace,
                                      size_t workspace_bytes, unsigned flags, void* stream);
QMM_API int qmm_bf16_matmul_small_m(const uint16_t* x, const uint16_t* w, uint16_t* y, int64_t M,
                                    int64_t N, int64_t K, void* stream);

/* ---------------------------------------------------------------------------
 * StableHLO front end: text in, launch plan out.
 *
 * qmm_plan_compile reads the textual StableHLO of a module (the form
 * jax.jit(f).lower(...).as_text() prints), matches every dot_general with the
 * dequantisation chain that feeds it and builds one kernel launch per match;
 * it stands where the reference parses and plans a program
 * (src/pjrt_plugin/core/stablehlo_parser.mm:521-586,
 *  src/pjrt_plugin/core/mps_executable.mm:7627-9008; pattern fusions
 *  :1214-1326).  Ops that no match absorbs run as standalone GPU kernels when
 * they belong to the supported set (convert, multiply, subtract, add, and,
 * shift_right_logical, broadcast_in_dim, reshape, transpose, slice,
 * concatenate, constant, dot / dot_general without batch dimensions); any
 * other op makes compilation fail with QMM_ERR_UNSUPPORTED and a message
 * naming the op and its line, as the reference reports unsupported ops
 * (src/pjrt_plugin/api/pjrt_client.cc:211-220).  Nothing is executed on the
 * CPU.  Dense constants become extra arguments owned by the plan (device
 * copies are made on the first execution on a device, which therefore
 * allocates; do it outside a stream capture).
 * qmm_plan_trace returns one JSON line per decision ("QMM_PLAN_JSON:{...}":
 * "fused" with the kernel, "not_fused" with the op — and the reason for a dot
 * that no pattern took —, "plan" with the step counts; also written to stderr
 * when QMM_TRACE_PLAN is set), the counterpart of the reference's
 * JAX_METALLIB_TRACE_PLAN output (mps_executable.mm:7925-7961).
 * qmm_plan_execute takes the device pointers of @main's arguments and results
 * in declaration order and a 256-byte aligned workspace of
 * qmm_plan_workspace_bytes (kernel scratch and the temporaries of unfused
 * ops; its first use must find it zero-filled). */
typedef struct qmm_plan qmm_plan;
QMM_API int qmm_plan_compile(const char* stablehlo_text, size_t length, qmm_plan** plan);
QMM_API void qmm_plan_destroy(qmm_plan* plan);
QMM_API int qmm_plan_num_steps(const qmm_plan* plan);
QMM_API int qmm_plan_num_fused_steps(const qmm_plan* plan); /* steps that are fused matmul kernels */
QMM_API int qmm_plan_num_args(const qmm_plan* plan);
QMM_API int qmm_plan_num_results(const qmm_plan* plan);
QMM_API size_t qmm_plan_workspace_bytes(const qmm_plan* plan);
/* Element type (a qmm_dtype, or -1 for a type the library has no tag for), rank
 * and dimensions of @main's arguments and results.  *rank carries the capacity
 * of dims on entry and the rank on return; dims may be NULL. */
QMM_API int qmm_plan_arg_info(const qmm_plan* plan, int index, int* dtype, int64_t* dims, int* rank);
QMM_API int qmm_plan_result_info(const qmm_plan* plan, int index, int* dtype, int64_t* dims, int* rank);
/* Module symbol, mhlo.num_replicas / mhlo.num_partitions, and the operation
 * count (2 M N K summed over the fused matmuls) of the plan. */
QMM_API const char* qmm_plan_name(const qmm_plan* plan);
QMM_API int qmm_plan_num_replicas(const qmm_plan* plan);
QMM_API int qmm_plan_num_partitions(const qmm_plan* plan);
QMM_API double qmm_plan_flops(const qmm_plan* plan);
QMM_API size_t qmm_plan_trace(const qmm_plan* plan, char* buf, size_t cap);
QMM_API int qmm_plan_execute(const qmm_plan* plan, const void* const* args, int num_args,
                             void* const* results, int num_results, void* workspace,
                             size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QMM_H_ */
