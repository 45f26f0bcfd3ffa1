/* libb200ait: C ABI of the per-op kernels (sm_100a) behind the AITemplate op API.
 *
 * Every function returns 0 on success and non-zero on failure; the text of the failure is
 * available from b200ait_last_error() on the calling thread. Pointers are device pointers unless
 * stated otherwise; `stream` is a cudaStream_t (NULL = legacy default stream). No function
 * allocates or synchronises unless its comment says so. Zero-size problems launch nothing.
 *
 * The reference generates one C++ function per op instance from Jinja templates; each entry
 * point below names the template whose signature it follows (paths relative to the reference
 * repository root).
 */
#ifndef B200AIT_H_
#define B200AIT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200ait_stream_t;

/* dtype codes are the values of AITemplateDtype (static/include/model_interface.h:70-78) */
enum { B200AIT_HALF = 1, B200AIT_FLOAT = 2, B200AIT_BFLOAT16 = 6 };

/* epilogue = u1 | b1 << 4 | b2 << 6 | u2 << 8 :  y = U2(B2(B1(U1(alpha*acc + bias), D0), D1))
 * (python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_elementwise.py:34-53) */
enum {
  B200AIT_UNARY_IDENTITY = 0, B200AIT_UNARY_RELU = 1, B200AIT_UNARY_GELU = 2, B200AIT_UNARY_FAST_GELU = 3,
  B200AIT_UNARY_SIGMOID = 4, B200AIT_UNARY_TANH = 5, B200AIT_UNARY_SWISH = 6, B200AIT_UNARY_HARDSWISH = 7
};
enum { B200AIT_BINARY_NONE = 0, B200AIT_BINARY_ADD = 1, B200AIT_BINARY_MUL = 2 };
/* store modes of b200ait_gemm_rcr */
enum { B200AIT_STORE_ROW_MAJOR = 0, B200AIT_STORE_PERMUTE_20314 = 1, B200AIT_STORE_PERMUTE_0213 = 2 };

const char* b200ait_last_error(void);
int b200ait_version(void);
/* Synchronises the device, then reads and clears the kernel status word (0 = clean). A non-zero
 * value means a bounded wait inside a kernel gave up and that kernel's output is invalid. */
int b200ait_device_status(int* status_out);
/* Number of kernels the library has launched in this process so far (a launch made during a stream
 * capture counts once, at capture). No counterpart in the reference; used to report launch counts. */
int b200ait_kernel_launch_count(int64_t* count_out);
/* Exercises the bounded wait of the pipeline kernels: one CTA waits, with a 1 ms limit, on an mbarrier
 * nobody arrives on, gives up and returns. out[0] = result of that wait (0 = gave up), out[1] = result of a
 * later wait in the same CTA (0 = returned at once), out[2] = ns spent. Leaves code 5 in the status word
 * for b200ait_device_status to report and clear. The reference has no device-side waits to bound
 * (its kernels are single-pass CUTLASS launches); host-side it maps to DeviceCheckLastError,
 * static/include/model.h:22-32. */
int b200ait_selftest_bounded_wait(int64_t* out, void* stream);

/* Generic GEMM: c[b] = epilogue(alpha * a[b] . b[b]^T + bias, d0, d1); a [batch, m, k] (row stride lda),
 * b [batch, n, k] (row stride ldb), c / d0 / d1 [batch, m, n] (row strides ldc / ldd). A batch stride
 * of 0 broadcasts that operand. tile_n = 0 lets the library choose; else 64, 128 or 256 (128 x tile_n tiles,
 * one CTA each) or 512 (256 x 256 tiles, each computed by a pair of CTAs with cta_group::2 MMAs).
 * With tile_n = 0 and split_k = 0 an unbatched problem with few rows or few output tiles is served by the
 * weight-streaming kernels instead of the tiles: m <= 4 by one that multiplies on the FMA pipe; otherwise, against
 * n >= 128 and k >= 256, by one that puts the weight rows on the MMA rows, takes the rows of x in groups of 16 to 256
 * and splits k across a thread-block cluster. Which problems it takes is planned from their size: weights above 16 MB
 * up to m = 256 (larger m while k >= 2048 and ceil(m / 256) * ceil(n / 128) <= 32); smaller weights up to m = 1024
 * and 64 output tiles of 128 x 128 (48 with an added residual, 32 with any other epilogue beyond bias + relu). Neither needs the workspace.
 * workspace / workspace_bytes / split_k: see b200ait_gemm_rcr_workspace_bytes below.
 * Replaces python/aitemplate/backend/cuda/gemm_universal/common.py:130-617 (CUTLASS instantiation). */
int b200ait_gemm_rcr(const void* a, const void* b, const void* bias, const void* d0, const void* d1, void* c,
                     int64_t batch, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                     int64_t ldd, int64_t a_batch_stride, int64_t b_batch_stride, int64_t c_batch_stride,
                     int64_t d_batch_stride, int epilogue, int dtype, float alpha, int store_mode, int64_t t1,
                     int64_t t2, int64_t t3, int tile_n, void* workspace, int64_t workspace_bytes, int split_k,
                     b200ait_stream_t stream);
/* Split-K (reference: split_k search, python/aitemplate/compiler/ops/gemm_universal/gemm_common.py:579-594):
 * when the output tiles cannot fill the GPU and K is deep, K is divided among CTAs that write fp32 partial
 * sums into `workspace` ([splits, batch, m, n] floats) and a second kernel reduces them and applies the
 * epilogue. split_k: 0 = library chooses, 1 = off, n = at most n. A null workspace disables splitting.
 * b200ait_gemm_rcr_workspace_bytes reports what the library would use for a problem. */
int b200ait_gemm_rcr_workspace_bytes(int64_t batch, int64_t m, int64_t n, int64_t k, int tile_n, int split_k,
                                     int64_t* bytes_out);
/* b200ait_gemm_rcr with B stored [batch, k, n] (n contiguous, row stride ldb): gemm_rrr / gemm_rrr_bias / bmm_rrr
 * (python/aitemplate/compiler/ops/gemm_universal/gemm_rrr.py:26-80, bmm_xxx.py:223-260). No permuted store. */
int b200ait_gemm_rrr(const void* a, const void* b, const void* bias, const void* d0, const void* d1, void* c,
                     int64_t batch, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                     int64_t ldd, int64_t a_batch_stride, int64_t b_batch_stride, int64_t c_batch_stride,
                     int64_t d_batch_stride, int epilogue, int dtype, float alpha, int tile_n, void* workspace,
                     int64_t workspace_bytes, int split_k, b200ait_stream_t stream);
/* bmm_rcr_permute / bmm_rrr_permute (python/aitemplate/compiler/ops/gemm_universal/bmm_rcr_permute.py:28-116,
 * bmm_rrr_permute.py; generated function python/aitemplate/backend/cuda/gemm_universal/bmm_common.py:56-81 with the
 * Permute4DBMM_0213 epilogue): c[b] = alpha * a[b] @ b[b]^T for b [batch, n, k] (b_row_major = 0), or a[b] @ b[b]
 * for b [batch, k, n] (b_row_major = 1), stored as [batch / d1, d1, m, n].permute(0, 2, 1, 3): c has the shape
 * [batch / d1, m, d1, n]. A batch stride of 0 broadcasts that operand; batch must be a multiple of d1. */
int b200ait_bmm_permute0213(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                            int64_t a_batch_stride, int64_t b_batch_stride, int64_t d1, int b_row_major, int dtype,
                            float alpha, int tile_n, b200ait_stream_t stream);
/* No counterpart in the reference (it is single-GPU: no communication backend anywhere under python/aitemplate
 * or static/). The same GEMM with its result written to num_out buffers of identical shape and strides
 * (1 <= num_out <= 8) by the epilogue's TMA stores. outs[0] is normally this GPU's buffer and the others
 * peer-mapped pointers into other GPUs' buffers (b200ait_peer_open), so a rank that computes one column
 * block of Y = X W^T places it in every rank's full Y while it computes the next tile, instead of an all-gather
 * pass afterwards. Never splits K; needs N and ldc multiples of 8 and 16-byte aligned pointers. */
int b200ait_gemm_rcr_multi_out(const void* a, const void* b, const void* bias, const void* d0, void* const* outs,
                               int num_out, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                               int64_t ldd, int epilogue, int dtype, float alpha, int tile_n,
                               b200ait_stream_t stream);
/* Device buffers that other processes of the node can open (CUDA IPC; one process per GPU).
 * b200ait_peer_alloc returns the pointer and a 64-byte handle to ship to the peers; b200ait_peer_open turns a
 * received handle into a pointer valid in this process; close what was opened, free what was allocated. */
int b200ait_peer_alloc(int64_t bytes, void** ptr_out, void* handle64_out);
int b200ait_peer_open(const void* handle64, void** ptr_out);
int b200ait_peer_close(void* opened_ptr);
int b200ait_peer_free(void* allocated_ptr);
/* No counterpart in the reference. b200ait_gemm_rcr for callers that cannot allocate device memory
 * (a serving process living inside a pre-sized pool, a framework allocator that owns the device, a
 * path that must avoid driver allocation calls): the split-K partial sums and the kernel status
 * word live in a 16 MiB + 256 B array inside the library image, so this call runs no cudaMalloc /
 * cudaFree. Problems whose two-split partial sums exceed the array (2 * batch * m * n * 4 bytes >
 * 16 MiB) are rejected. The first call on a device does one-time set-up and belongs outside any
 * stream capture; all calls on a device share the array, so keep them stream-ordered (calls that
 * overlap on the GPU race). status_out: optional device int that receives the status word. */
int b200ait_gemm_rcr_static_scratch(const void* a, const void* b, const void* bias, const void* d0,
                                    const void* d1, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                                    int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, int64_t a_batch_stride,
                                    int64_t b_batch_stride, int64_t c_batch_stride, int64_t d_batch_stride,
                                    int epilogue, int dtype, float alpha, int store_mode, int64_t t1, int64_t t2,
                                    int64_t t3, int tile_n, int split_k, int* status_out, b200ait_stream_t stream);

/* fp16 entry points with the reference's generated signatures. workspace / split_k are accepted
 * and ignored. *c_dim0, *c_dim1 are written.
 * gemm_rcr: python/aitemplate/backend/cuda/gemm_universal/common.py:172-198 */
int b200ait_gemm_rcr_plain(void* a, void* b, void* c, uint8_t* workspace, int split_k, int64_t* a_dim0,
                           int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, int64_t* c_dim0, int64_t* c_dim1,
                           b200ait_stream_t stream);
/* gemm_rcr_bias + activation: python/aitemplate/backend/cuda/gemm_universal/common_bias.py:77-97 */
#define B200AIT_DECL_GEMM_BIAS(NAME)                                                                          \
  int b200ait_##NAME(void* a, void* b, void* bias, void* c, uint8_t* workspace, int split_k, int64_t* a_dim0, \
                     int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, int64_t* c_dim0, int64_t* c_dim1,     \
                     b200ait_stream_t stream);
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_relu)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_gelu)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_fast_gelu)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_sigmoid)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_tanh)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_swish)
B200AIT_DECL_GEMM_BIAS(gemm_rcr_bias_hardswish)
#undef B200AIT_DECL_GEMM_BIAS
/* gemm_rcr_bias + residual(s): python/aitemplate/backend/cuda/gemm_universal/common_bias_broadcast.py:276-305 */
#define B200AIT_DECL_GEMM_BIAS_D0(NAME)                                                                        \
  int b200ait_##NAME(void* a, void* b, void* bias, void* d0, void* c, uint8_t* workspace, int split_k,         \
                     int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1, int64_t* c_dim0,      \
                     int64_t* c_dim1, b200ait_stream_t stream);
#define B200AIT_DECL_GEMM_BIAS_D0_D1(NAME)                                                                     \
  int b200ait_##NAME(void* a, void* b, void* bias, void* d0, void* d1, void* c, uint8_t* workspace,            \
                     int split_k, int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1,          \
                     int64_t* c_dim0, int64_t* c_dim1, b200ait_stream_t stream);
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_add)
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_add_relu)
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_mul)
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_mul_tanh)
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_sigmoid_mul)
B200AIT_DECL_GEMM_BIAS_D0(gemm_rcr_bias_sigmoid_mul_tanh)
B200AIT_DECL_GEMM_BIAS_D0_D1(gemm_rcr_bias_add_add)
B200AIT_DECL_GEMM_BIAS_D0_D1(gemm_rcr_bias_add_add_relu)
B200AIT_DECL_GEMM_BIAS_D0_D1(gemm_rcr_bias_mul_add)
#undef B200AIT_DECL_GEMM_BIAS_D0
#undef B200AIT_DECL_GEMM_BIAS_D0_D1
/* gemm_rcr_bias_permute, layout "20314", shape (t1, t2, t3): result [M, N] is stored as
 * [t2, M/t1, t3, t1, N/(t2*t3)] (python/aitemplate/backend/cuda/gemm_universal/gemm_rcr_bias_permute.py:55-95) */
int b200ait_gemm_rcr_bias_permute(void* a, void* b, void* bias, void* c, uint8_t* workspace, int split_k,
                                  int64_t* a_dim0, int64_t* a_dim1, int64_t* b_dim0, int64_t* b_dim1,
                                  int64_t* c_dim0, int64_t* c_dim1, int64_t t1, int64_t t2, int64_t t3,
                                  b200ait_stream_t stream);
/* bmm_rcr: python/aitemplate/backend/cuda/gemm_universal/bmm_common.py:56-81 */
int b200ait_bmm_rcr(void* a, void* b, void* c, uint8_t* workspace, int64_t* a_dim0, int64_t* a_dim1,
                    int64_t* a_dim2, int64_t* b_dim0, int64_t* b_dim1, int64_t* b_dim2, int64_t* c_dim0,
                    int64_t* c_dim1, int64_t* c_dim2, b200ait_stream_t stream);

/* mem_eff_attention: q [B,H,Sq,D], k [B,H,Skv,D], v [B,H,Skv,Dv] -> output [B,Sq,H,Dv]
 * (python/aitemplate/backend/cuda/attention/mem_eff_attention.py:632-654). lengths_kv / lengths_q: NULL, or
 * batch_size int32 values on the device: batch b attends to its first lengths_kv[b] keys, and only its first
 * lengths_q[b] query rows are computed and written (static/include/kernels/mem_eff_attention/kernel_forward.h:183-197);
 * a batch with lengths_kv[b] = 0 comes out NaN, as it does there. */
int b200ait_mem_eff_attention(void* output, const void* query, const void* key, const void* value,
                              int64_t batch_size, int64_t seq_len_kv, int64_t seq_len_q, int num_heads,
                              int head_size, int head_size_v, float softmax_scale, int is_causal,
                              const int32_t* lengths_kv, const int32_t* lengths_q, int dtype,
                              b200ait_stream_t stream);

/* mem_eff_attention whose q, k, v are strided views: each is addressed as [batch, head, row, channel] with unit
 * channel stride and the three element strides {row, head, batch} given, e.g. {H*D, D, S*H*D} reads a [B, S, H, D]
 * projection output in place. Strides: positive multiples of 8 elements; head sizes: multiples of 8, at most 128.
 * Output [B, Sq, H, Dv] contiguous. Counterpart of the q/k/v strides the reference passes to its kernel through
 * the op's input TensorAccessors (python/aitemplate/backend/cuda/attention/mem_eff_attention.py:160-171). */
int b200ait_mem_eff_attention_strided(void* output, const void* query, const void* key, const void* value,
                                      int64_t batch_size, int64_t seq_len_kv, int64_t seq_len_q, int num_heads,
                                      int head_size, int head_size_v, const int64_t* q_strides,
                                      const int64_t* k_strides, const int64_t* v_strides, float softmax_scale,
                                      int is_causal, int dtype, b200ait_stream_t stream);

/* flash_attention: qkv [total, 3, num_heads, head_size] (all sequences' rows back to back), cu_seqlens int32
 * [batch_size + 1] on the device, output [total, num_heads, head_size]; sequence b attends within rows
 * cu_seqlens[b] .. cu_seqlens[b+1]. seq_len = (an upper bound of) the longest sequence, total_rows = row extent of
 * qkv. softmax_lse, o_tmp and loop belong to the reference kernel and are ignored; p_dropout must be 0.
 * (python/aitemplate/backend/cuda/attention/flash_attention.py:199-215; total_rows and dtype are appended) */
int b200ait_flash_attention(void* output, const void* qkv, const int* cu_seqlens, float* softmax_lse, float* o_tmp,
                            int batch_size, int seq_len, int num_heads, int head_size, float p_dropout,
                            float softmax_scale, int is_causal, int loop, int64_t total_rows, int dtype,
                            b200ait_stream_t stream);

/* layernorm over the last n elements of each of m rows; gamma / beta may be NULL; a row stride of 0
 * means n (python/aitemplate/backend/cuda/layernorm_sigmoid_mul/layernorm_sigmoid_mul.py:72-83) */
int b200ait_layernorm(void* out, const void* in, const void* gamma, const void* beta, int64_t m, int64_t n,
                      float eps, int64_t in_row_stride, int64_t out_row_stride, int dtype,
                      b200ait_stream_t stream);

/* softmax over the middle axis of a tensor viewed as [outer, k, inner]
 * (python/aitemplate/backend/cuda/softmax/softmax.py:142-153) */
int b200ait_softmax(const void* in, void* out, int64_t outer, int64_t k, int64_t inner, int dtype,
                    b200ait_stream_t stream);

/* concatenate / split (python/aitemplate/backend/common/concatenate_common.py:29-48,
 * split_common.py:21-40). inputs / input_shapes / masks / shapes are HOST arrays. */
int b200ait_concatenate(void* output, int64_t* output_shape, const void* const* inputs,
                        const int64_t* const* input_shapes, const uint8_t* input_masks, int64_t concat_dim,
                        int64_t rank, int64_t num_inputs, int64_t elem_size, b200ait_stream_t stream);
int b200ait_split(void* const* outputs, const uint8_t* output_masks, const void* input, const int64_t* input_shape,
                  int64_t num_splits, const int64_t* split_sizes, int64_t split_dim, int64_t rank,
                  int64_t elem_size, b200ait_stream_t stream);

/* output = input.permute(dims), made contiguous (python/aitemplate/backend/cuda/tensor/permute.cuh:227-389) */
int b200ait_permute(const void* input, void* output, const int64_t* input_shape, const int64_t* dims, int64_t rank,
                    int64_t elem_size, b200ait_stream_t stream);

/* element-wise chain with broadcasting (python/aitemplate/backend/common/elementwise_common.py:201-264):
 * acc = inputs[0]; acc = ops[s](acc, operand) for each step; operand_index[s] >= 0 selects an input,
 * -1 the scalar constants[s], -2 nothing (unary op). Op codes: 1 add, 2 sub, 3 mul, 4 div, 5 rsub,
 * 6 rdiv, 7 max, 8 min, 16 relu, 17 gelu, 18 fast_gelu, 19 sigmoid, 20 tanh, 21 silu, 22 neg, 23 abs,
 * 24 exp, 25 sqrt, 26 hardswish. */
int b200ait_elementwise(void* output, const int64_t* out_shape, int64_t rank, const void* const* inputs,
                        const int64_t* const* input_shapes, int64_t num_inputs, const int* ops,
                        const int* operand_index, const float* constants, int64_t num_steps, int dtype,
                        b200ait_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200AIT_H_ */
