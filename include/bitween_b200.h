/*
 * bitween_b200.h -- C ABI of libbitween_b200.so, the sm_100a replacement for the
 * reference's kernel directory (bitween/kernels/) and for the eager tensor code on its
 * RTN quantize / QuantizedLinear forward path.
 *
 * Conventions for every entry point:
 *   - plain pointers and sizes only; every pointer is DEVICE memory owned by the caller
 *     unless the name says host; nothing the caller sees is allocated here (the one exception
 *     is bw_peer_alloc / bw_peer_free: memory that other processes map needs its own allocation)
 *   - asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default stream),
 *     on the CUDA device that is current in the calling thread
 *   - returns a bw_status (0 = BW_OK); never throws, aborts or traps
 *   - tensors are dense row-major
 *
 * Packed-weight wire format (identical to the reference, bitween/functional.py:31-43):
 *   vpi = 32 / bits codes per int32 word; qweight[n][j] holds the codes of
 *   k = j*vpi .. j*vpi+vpi-1, code i in bits [i*bits, (i+1)*bits); codes are unsigned
 *   (0 .. 2^bits-1) inside a signed int32 container; scale[n][k / group_size],
 *   zero_point[n][k / group_size]; dequantized weight = scale * (code - zero_point).
 */
#ifndef BITWEEN_B200_H_
#define BITWEEN_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BW_API __attribute__((visibility("default")))
#else
#define BW_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BW_F32 = 0,
    BW_F16 = 1,
    BW_BF16 = 2,
    BW_I32 = 3
} bw_dtype;

typedef enum {
    BW_OK = 0,
    BW_ERR_BITS = 1,        /* bits not in {2,4,8}            (AssertionError in the reference) */
    BW_ERR_GROUP = 2,       /* group_size < 1 or K % group_size != 0   (ValueError)            */
    BW_ERR_SHAPE = 3,       /* negative size, K % (32/bits) != 0, size overflow                */
    BW_ERR_DTYPE = 4,       /* dtype code not accepted by this argument                        */
    BW_ERR_ALIGN = 5,       /* pointer not aligned for its element type                        */
    BW_ERR_NULL = 6,        /* required pointer is NULL                                        */
    BW_ERR_WORKSPACE = 7,   /* workspace smaller than bw_qmatmul_workspace_bytes()             */
    BW_ERR_CUDA = 8,        /* a CUDA runtime call failed; see bw_last_cuda_error()            */
    BW_ERR_UNSUPPORTED = 9, /* valid request this build has no kernel for                      */
    BW_ERR_TIMEOUT = 10,    /* a bounded device-side wait ran out (reported via status word)   */
    BW_ERR_TOO_LARGE = 11   /* request exceeds the fixed scratch of bw_qmatmul_noalloc         */
} bw_status;

/* flags for bw_rtn_quantize_pack */
#define BW_RTN_UPCAST_F32 1u /* 16-bit weights: up-cast each element to fp32 and do all
                                arithmetic in fp32, i.e. what QuantizedLinear.from_float gets
                                from `deepcopy(layer).to(float32)` (bitween/modules.py:191)   */
#define BW_RTN_TMA_STREAM 2u /* large inputs: stream the weights through shared memory with bulk
                                asynchronous copies instead of register loads; same results    */

/*
 * RTN group-wise quantize + pack.  Replaces bitween/functional.py:3-45 (quantize_rtn): per
 * group of `group_size` consecutive input-dim elements of each row, min/max, scale =
 * max((max-min)/Qmax, 1e-8), zero_point = clamp(round(-min/scale), 0, Qmax), codes =
 * clamp(round(w/scale + zero_point), 0, Qmax), packed into int32 words.  Every operation
 * is rounded exactly as torch's op-by-op evaluation in the weight dtype, so the outputs
 * are bit-identical to the reference run on CPU.
 *
 *   w          [N,K]            BW_F32 | BW_F16 | BW_BF16
 *   qweight    [N,K*bits/32]    int32 out
 *   scale      [N,K/group_size] out; BW_F32 | BW_F16 | BW_BF16.  The reference returns the
 *                               weight dtype; BW_F16 applies the fp32->fp16 copy_ cast of
 *                               QuantizedLinear.from_float (bitween/modules.py:208) in place.
 *   zero_point [N,K/group_size] out; BW_I32 (reference API) or BW_F16 (module buffer,
 *                               bitween/modules.py:209)
 */
BW_API int bw_rtn_quantize_pack(const void *w, int w_dtype, int64_t N, int64_t K, int bits,
                         int group_size, int32_t *qweight, void *scale, int scale_dtype,
                         void *zero_point, int zp_dtype, unsigned flags, void *stream);

/*
 * RTN quantize + pack of several weight matrices in one call: the per-layer loops of the
 * reference (bitween/quantizer/quantizer.py:72-80 over a model, bitween/gradual/base_wrapper.py:
 * 300-311 over a decoder block) call quantize_rtn once per layer; for the handful of linears of
 * a block the launches, not the kernel, are the cost.  All matrices share the weight dtype, bit
 * width, group size and output dtypes; shapes differ.  One kernel is launched when every matrix
 * takes the vector path (group_size a power-of-two multiple of the elements in 16 bytes, up to
 * 32 such chunks; weights 16-byte and packed words 8-byte aligned), else one per matrix.
 *   jobs       HOST array of njobs entries (pageable is fine; read before the call returns)
 *   table_dev  device scratch of bw_rtn_batch_table_bytes(njobs) bytes for the job table, which
 *              the call copies there with one asynchronous copy on `stream`; must stay untouched
 *              until the kernel has run.  Not for use inside a stream capture.
 * Results per matrix are those of bw_rtn_quantize_pack.
 */
typedef struct {
    const void *w;       /* [N,K] weights                      */
    int32_t *qweight;    /* [N,K*bits/32] out                  */
    void *scale;         /* [N,K/group_size] out               */
    void *zero_point;    /* [N,K/group_size] out               */
    int64_t N, K;
} bw_rtn_job;
BW_API size_t bw_rtn_batch_table_bytes(int njobs);
BW_API int bw_rtn_quantize_pack_batch(const bw_rtn_job *jobs, int njobs, int w_dtype, int bits, int group_size,
                               int scale_dtype, int zp_dtype, unsigned flags, void *table_dev,
                               size_t table_bytes, void *stream);

/*
 * Dequantize packed weights: out[n][k] = out_dtype( float(scale) * (float(code) - float(zp)) ).
 * With BW_F32 scale / BW_I32 zero_point / BW_F32 out it replaces bitween/functional.py:47-71
 * (dequantize_rtn); with BW_F16 scale and zero_point and BW_F16 out it replaces the Triton
 * kernel bitween/modules.py:10-58; it is also the weight reconstruction of the backward
 * pass (bitween/modules.py:121-135).
 *   scale: BW_F32|BW_F16|BW_BF16   zero_point: BW_I32|BW_F32|BW_F16|BW_BF16
 *   out  : BW_F32|BW_F16|BW_BF16
 */
BW_API int bw_dequantize(const int32_t *qweight, const void *scale, int scale_dtype,
                  const void *zero_point, int zp_dtype, int64_t N, int64_t K, int bits,
                  int group_size, void *out, int out_dtype, void *stream);

/*
 * QuantizedLinear forward: out[m][n] = sum_k x[m][k] * W[n][k] (+ bias[n]),
 * W[n][k] = fp16( scale * (code - zero_point) ).  Replaces
 * QuantizedLinearFunction.forward, bitween/modules.py:61-106 (Triton dequantize to a
 * temporary fp16 [N,K] + torch.matmul + bias add), and is the body of the
 * `quantized_matmul_cuda(x, qweight, scale, zero_point, bias, bits, group_size)` symbol the
 * reference's scripts import (main.py:401,433).
 *
 *   x        [M,K]  BW_F16 | BW_BF16 | BW_F32; cast to fp16 first, as bitween/modules.py:74
 *   qweight  [N,K*bits/32] int32
 *   scale    [N,K/group_size] fp16          (module buffer dtype, bitween/modules.py:177)
 *   zero_point [N,K/group_size] fp16, integer-valued in [0,255]  (bitween/modules.py:178)
 *   bias     [N] fp16 or NULL
 *   out      [M,N]  BW_F16: fp16(fp16(acc) + bias), the reference's two roundings
 *                   (bitween/modules.py:97,101); BW_BF16: bf16(acc + bias);
 *                   BW_F32: acc + bias with no 16-bit rounding (fp32-accumulate checks)
 *   workspace       device scratch of at least bw_qmatmul_workspace_bytes(...) bytes, or
 *                   NULL when that is 0.  Calls that overlap on the GPU must not share it,
 *                   and a workspace address identifies the caller to the library (the
 *                   decode kernel keeps its row-block counters per workspace address, for
 *                   up to 64 addresses per device; further ones use the cluster kernel).
 *                   Make the first call with a new workspace address outside a stream
 *                   capture (it looks up the address of the library's counter array).
 * Accumulation is fp32.  The kernel is chosen from M and the layout: up to 32 tokens run on
 * the persistent TMA-fed decode kernel (one launch; needs K/group_size to be a multiple of 8
 * and 16-byte aligned rows, else the cluster split-K streaming kernel runs), more on the
 * tcgen05 tensor-core GEMM; unusual group sizes run on a slower general kernel, never on the
 * CPU.  The kernels are launched with programmatic dependent launch and fetch packed weights,
 * scales and zero points BEFORE waiting for the preceding kernel of the stream (only the
 * activations are read after it): qweight, scale and zero_point must not be written by the one
 * or two kernels that precede the call on its stream -- put an event or any non-library kernel
 * between a weight update and the call.
 * bw_qmatmul_workspace_bytes: the prepared activations of the cluster kernel (K rounded
 * up to a k-chunk x 8*ceil(min(M,64)/8) x 2 bytes), the fp16 cast of the activations for the
 * GEMM (M*K*2), or the decode kernel's row-block shares (320 x 8*ceil(M/8) x 128 x 4 bytes),
 * whichever the call may need most.
 */
BW_API size_t bw_qmatmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int bits, int group_size);
/* Same query for given activations: fp16 activations that start on a 16-byte boundary need no
 * cast for the tensor-core GEMM (x_align = the largest power of two, up to 16, dividing the
 * address of x), so large prefill calls need no workspace at all. */
BW_API size_t bw_qmatmul_workspace_bytes_for(int64_t M, int64_t N, int64_t K, int bits, int group_size,
                                      int x_dtype, int x_align);

BW_API int bw_qmatmul(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K,
               const int32_t *qweight, const void *scale, const void *zero_point,
               const void *bias, void *out, int out_dtype, int bits, int group_size,
               void *workspace, size_t workspace_bytes, void *stream);

/*
 * bw_qmatmul with the operations that follow the linear in a decoder block fused into the
 * kernels' output stage: activation and residual add.  The reference runs them -- and even the
 * bias add (bitween/modules.py:100-101) -- as separate elementwise kernels over [M, N]; the
 * block structure they come from is the one bitween/gradual/utils.py:292-392 walks (OPT:
 * fc1 -> ReLU -> fc2 -> + residual).
 *   out = act( fp16(fp16(acc) + bias) ) + residual      (each step rounded to fp16 for BW_F16 out,
 *                                                         like the separate torch ops; fp32 math
 *                                                         with one final rounding otherwise)
 *   ep->activation  BW_ACT_NONE | BW_ACT_RELU | BW_ACT_SILU_MUL
 *   ep->residual    [M,N] fp16 or NULL; may alias `out`
 * ep == NULL is bw_qmatmul.
 * BW_ACT_SILU_MUL is the gated feed-forward (Llama gate / up) as ONE [2*ffn, K] packed GEMM: row 2i
 * of the packed weight (and of scale, zero_point, bias) is gate row i, row 2i+1 is up row i, and
 *   out[m, i] = silu(lin[m, 2i]) * lin[m, 2i+1] (+ residual[m, i]),    out and residual are [M, N/2]
 * with lin rounded as the plain call rounds it, silu evaluated in fp32, every step rounded to fp16
 * for BW_F16 out (fp32 math with one final rounding otherwise).  N must be a multiple of 4.  Served
 * by the decode kernel (M <= 32) and the tensor-core kernel; layouts neither can take return
 * BW_ERR_UNSUPPORTED with nothing launched (the caller runs the plain call and its own elementwise op).
 */
#define BW_ACT_NONE 0
#define BW_ACT_RELU 1
#define BW_ACT_SILU_MUL 2
typedef struct {
    int activation;
    const void *residual;
} bw_epilogue;
BW_API int bw_qmatmul_fused(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K,
                     const int32_t *qweight, const void *scale, const void *zero_point,
                     const void *bias, void *out, int out_dtype, int bits, int group_size,
                     const bw_epilogue *ep, void *workspace, size_t workspace_bytes, void *stream);

/*
 * bw_qmatmul for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its forward allocates a temporary fp16 [N,K] on every call.)
 *
 * Who needs it: code that runs while a CUDA graph is being captured or inside a latency-bound
 * serving loop where allocator calls are forbidden after start-up, and host plugins that are
 * handed only their input and output buffers.  Instead of a caller-supplied workspace the
 * prepared activations go to a 2 MiB array that is part of the library image (every GPU that
 * loads the library holds it until the process exits).  The call makes no cudaMalloc /
 * cudaFree and uses no allocating library routine; the caller still owns x, the packed
 * weights and out.
 *
 * Limit: what the kernel that runs needs from the array must not exceed
 * bw_qmatmul_noalloc_max_scratch_bytes() (2 MiB); otherwise BW_ERR_TOO_LARGE is returned and
 * nothing is launched.  Nothing is needed by the tensor-core GEMM (more than 32 tokens) on fp16
 * activations that start on a 16-byte boundary, nor by the general kernel (group sizes that
 * are not a power of two).  bf16 / fp32 (or misaligned) activations of the GEMM are cast to
 * fp16 into the array (M*K*2 bytes) when that fits; when it does not, and for up to 32 tokens,
 * the streaming kernel runs on blocks of at most 64 tokens and needs K (rounded up to a
 * k-chunk of 16*32/bits) * 8*ceil(min(M,64)/8) * 2 bytes: K <= 65536 for M <= 16, K <= 16384
 * for M >= 57.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) -- make that first call before starting a stream capture.
 * All calls on a device share the array and it keeps the last call's contents; every call
 * rewrites the part it reads (padding included), so nothing has to be cleared, but calls that
 * overlap on the GPU (different streams) race on it -- issue them on one stream.
 * Arguments and results are those of bw_qmatmul (same numerics; up to 32 tokens the sums may
 * be added in another order than bw_qmatmul's decode kernel does, so the last bit can differ).
 */
BW_API int bw_qmatmul_noalloc(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K,
                       const int32_t *qweight, const void *scale, const void *zero_point,
                       const void *bias, void *out, int out_dtype, int bits, int group_size,
                       void *stream);
BW_API size_t bw_qmatmul_noalloc_max_scratch_bytes(void);

/*
 * Same operator with HOST activations and HOST output (pinned memory for true overlap):
 * copies x to `x_dev`, runs bw_qmatmul, copies the result from `out_dev` to `out_host`, all
 * asynchronously on `stream`.  The packed weights stay resident on the device.  This is the
 * end-to-end call timed by the benchmark (host<->device copies inside the timed region).
 * Transfers of up to 4 MiB between 16-byte aligned buffers, the host one pinned, are made by a
 * small copy kernel through the pinned buffer's device mapping (no copy-engine set-up per
 * transfer, launch overlapped with the preceding kernel); anything else by cudaMemcpyAsync.
 * As with any asynchronous copy, the host may reuse x_host / read out_host only after the
 * stream has reached this call's end (event or synchronize).
 */
BW_API int bw_qmatmul_host(const void *x_host, int x_dtype, int64_t M, int64_t N, int64_t K,
                    const int32_t *qweight, const void *scale, const void *zero_point,
                    const void *bias, void *out_host, int out_dtype, int bits, int group_size,
                    void *x_dev, void *out_dev, void *workspace, size_t workspace_bytes,
                    void *stream);

/*
 * grad_input of QuantizedLinearFunction.backward (bitween/modules.py:108-141):
 * grad_in[m][k] = sum_n grad_out[m][n] * W[n][k], W = dtype( scale * (code - zero_point) )
 * evaluated in fp32 and cast to the gradient dtype (bitween/modules.py:131-139).
 *   grad_out [M,N], grad_in [M,K]: BW_F16 | BW_BF16 | BW_F32 (same dtype for both)
 */
BW_API int bw_qmatmul_grad_input(const void *grad_out, int grad_dtype, int64_t M, int64_t N, int64_t K,
                          const int32_t *qweight, const void *scale, const void *zero_point,
                          void *grad_in, int bits, int group_size, void *stream);

/*
 * Fake-quantized weights of the trainable mode: the elementwise part of
 * WrapperLinear._quantize_weight_with_learnable_params (bitween/wrapper.py:143-155), evaluated
 * on every training step there, as one pass.  The per-group scale and FLOAT zero point are
 * inputs (the caller derives them from the group minima / maxima and the learnable factors,
 * bitween/wrapper.py:127-140, on [N, K/group_size] tensors, where autograd tracks them):
 *     t    = w / scale + zero_point (+ value)
 *     w_q  = clamp(round_half_even(t), 0, 2^bits - 1)
 *     w_dq = scale * (w_q - zero_point)
 * in fp32, one rounding per operation in this order: bit-identical to the reference in fp32.
 *   w [N,K] BW_F32 | BW_F16 | BW_BF16 (up-cast exactly)   scale, zero_point [N,K/group_size] fp32
 *   value [N,K] of value_dtype (BW_F32 | BW_F16 | BW_BF16) or NULL
 *   w_dq [N,K] fp32 out           w_q [N,K] fp32 out or NULL
 */
BW_API int bw_fake_quant(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int group_size,
                  const float *scale, const float *zero_point, const void *value, int value_dtype,
                  float *w_dq, float *w_q, void *stream);

/*
 * bw_fake_quant when every tensor is 16-bit (16-bit weights and min/max tuning off: nothing promotes
 * the reference's arithmetic to fp32, bitween/wrapper.py:143-155 then rounds each intermediate to the
 * weight's dtype): w, scale, zero_point, value (or NULL), w_dq and w_q (or NULL) all have `dtype`
 * (BW_F16 | BW_BF16); every operation is rounded to it, bit-identical to the torch ops.
 */
BW_API int bw_fake_quant_native16(const void *w, int dtype, int64_t N, int64_t K, int bits, int group_size,
                           const void *scale, const void *zero_point, const void *value, void *w_dq,
                           void *w_q, void *stream);

/*
 * Backward of bw_fake_quant for the per-group parameters, as the reference's autograd graph
 * gives it (round() passes no gradient, bitween/wrapper.py:152-155):
 *     grad_scale      = sum over the group of grad_w_dq * (w_q - zero_point)
 *     grad_zero_point = -scale * sum over the group of grad_w_dq
 * w_q is recomputed from w (and value); `value` itself receives no gradient.  Sums are fp32 in
 * a fixed order (deterministic), not the order of torch's reduction: compare to ~1e-5 relative.
 * group_size must be 4 * 2^j <= 128 and w, value, grad_w_dq aligned to four elements,
 * else BW_ERR_GROUP / BW_ERR_ALIGN (the caller then uses its own reduction).
 *   grad_w_dq [N,K] fp32      grad_scale, grad_zero_point [N,K/group_size] fp32 out
 */
BW_API int bw_fake_quant_backward(const void *w, int w_dtype, int64_t N, int64_t K, int bits,
                           int group_size, const float *scale, const float *zero_point,
                           const void *value, int value_dtype, const float *grad_w_dq,
                           float *grad_scale, float *grad_zero_point, void *stream);

/*
 * All-reduce (sum) of the row-parallel layers' partial outputs over peer memory on one node,
 * without NCCL.  No counterpart in the reference (it is single-GPU); it replaces the
 * ncclAllReduce that follows o_proj / down_proj in the tensor-parallel layers of this library.
 * Set-up (once): every rank allocates its partial-sum buffers and one flag array with
 * bw_peer_alloc (cudaMalloc, zero-filled, plus a CUDA IPC handle of 64 bytes), the ranks exchange
 * the handles by any means, and every rank maps the others' with bw_peer_open.  Per call: the
 * rank's matmul writes its partial [count] fp16 values into its own buffer, then
 * bw_peer_allreduce_f16 (same stream) waits -- bounded, BW_ERR_TIMEOUT through bw_device_status --
 * until every rank's partial is complete, adds them in rank order in fp32 (the same bits on every
 * rank) and writes the fp16 sums to `out` (local memory).
 *   bufs, flags  host arrays of `world` device pointers: this process's mappings of rank r's
 *                partial buffer and flag array (bw_peer_flag_bytes() bytes, zero at start)
 *   state        bw_peer_state_bytes() bytes of local device memory, zero at start, one per flag array
 *   count        multiple of 8; all ranks call with the same count, in the same order
 * A buffer may be rewritten once ONE other call on the same flag array has been issued in
 * between (callers alternate between two partial buffers).  world <= 8, one process per GPU.
 * Plain peer loads and stores: no multicast object is created.
 */
BW_API int bw_peer_alloc(size_t bytes, void **ptr, unsigned char *ipc_handle_64);
BW_API int bw_peer_open(const unsigned char *ipc_handle_64, void **ptr);
BW_API int bw_peer_close(void *ptr);
BW_API int bw_peer_free(void *ptr);
BW_API size_t bw_peer_flag_bytes(void);
BW_API size_t bw_peer_state_bytes(void);
BW_API int bw_peer_allreduce_f16(const void *const *bufs, void *const *flags, int rank, int world, void *out,
                          int64_t count, void *state, void *stream);
/*
 * Two-shot form of the same all-reduce for many ranks: every rank sums one slice of the data and
 * publishes it in its result buffer (`results`: mappings of every rank's, ceil(count/world) values
 * rounded up to 8, alternated like the partial buffers), a second barrier, then every rank collects
 * the slices.  Per rank 2*(world-1)/world of the data crosses NVLink instead of (world-1) times
 * all of it.  Same sums, same bits as the one-shot form.
 */
BW_API int bw_peer_allreduce2_f16(const void *const *bufs, void *const *results, void *const *flags, int rank,
                           int world, void *out, int64_t count, void *state, void *stream);

/* Human-readable text for a bw_status. */
BW_API const char *bw_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
BW_API const char *bw_last_cuda_error(void);
/* Synchronizes the current device and reports whether any bounded device-side wait of the
 * library's kernels ran out since the last call (BW_ERR_TIMEOUT), clearing the flag. */
BW_API int bw_device_status(void);
/* Library version: major*10000 + minor*100 + patch. */
BW_API int bw_version(void);
/*
 * Self-test of the RTN kernel's division: it divides by one correctly rounded reciprocal per
 * group plus FMA corrections instead of a hardware division (bitween/functional.py:25-29 divides).
 * Runs both on n pseudo-random operand pairs (random and adversarial significands, the exponent
 * range of the fast path, the Qmax divisors) and returns the number of results that differ
 * from IEEE division in any bit (0 = exact), or -1 on a CUDA error.  Synchronous; allocates
 * and frees an 8-byte counter.
 */
BW_API long long bw_selftest_division(unsigned long long n, unsigned long long seed);
/* Name of the kernel the last bw_qmatmul call of this thread dispatched to (diagnostics). */
BW_API const char *bw_last_qmatmul_kernel(void);

#ifdef __cplusplus
}
#endif
#endif /* BITWEEN_B200_H_ */
