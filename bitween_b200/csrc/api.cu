// extern "C" entry points of libbitween_b200.so (declared in include/bitween_b200.h):
// argument validation, status codes and kernel dispatch.  No torch types, no allocation.
#include <cstdio>
#include <cstring>

#include "bw_common.cuh"

namespace bw {

static thread_local char g_cuda_error[256] = "";
static thread_local const char *g_last_kernel = "";
static thread_local Epilogue g_epilogue = {BW_ACT_NONE, nullptr};
Epilogue current_epilogue() { return g_epilogue; }

int record_cuda_error(cudaError_t e, const char *where) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
             cudaGetErrorString(e));
    (void)cudaGetLastError();  // clear the sticky-free error state for the next call
    return BW_ERR_CUDA;
}
void set_last_kernel(const char *name) { g_last_kernel = name; }

// implemented in the kernel translation units
int rtn_quantize_pack(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, int32_t *q,
                      void *scale, int scale_dtype, void *zp, int zp_dtype, unsigned flags,
                      cudaStream_t st);
size_t rtn_batch_table_bytes(int njobs);
int rtn_quantize_pack_batch(const bw_rtn_job *jobs, int njobs, int w_dtype, int bits, int g, int scale_dtype,
                            int zp_dtype, unsigned flags, void *table_dev, cudaStream_t st);
int dequantize(const int32_t *q, const void *scale, int scale_dtype, const void *zp, int zp_dtype,
               int64_t N, int64_t K, int bits, int g, void *out, int out_dtype, cudaStream_t st);
int qmatmul_smallm(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                   const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype,
                   int bits, int g, void *workspace, cudaStream_t st);
bool smallm_fast_path_ok(const void *x, int x_dtype, int64_t K, const int32_t *q, int bits, int g);
size_t smallm_workspace_bytes(int64_t M, int64_t K, int bits);
void set_smallm_tuning(int rt, int warps, int splits);
void set_smallm_pdl(int on);
int noalloc_scratch(void **ptr, size_t *bytes);
bool tc_path_ok(int64_t M, int64_t N, int64_t K, const int32_t *q, int bits, int g);
size_t tc_workspace_bytes(int64_t M, int64_t K);
int tc_device_status();
void set_tc_enabled(int on);
void set_tc_splits(int s);
int qmatmul_tc(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
               const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype, int bits,
               int g, void *workspace, cudaStream_t st);
bool decode_path_ok(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                    const void *scale, const void *zp, int bits, int g);
size_t decode_workspace_bytes(int64_t M, int64_t N, int64_t K, int bits);
int decode_device_status();
void set_decode_tuning(int enabled, int smem_kb, int max_ctas, int pdl);
int qmatmul_decode(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                   const __half *scale, const __half *zp, const __half *bias, void *out, int out_dtype,
                   int bits, int g, void *workspace, cudaStream_t st);
int fake_quant(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp,
               const void *value, int value_dtype, float *dq, float *wq, cudaStream_t st);
int fake_quant_native(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const void *scale, const void *zp,
                      const void *value, void *dq, void *wq, cudaStream_t st);
int fake_quant_backward(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int g, const float *scale, const float *zp,
                        const void *value, int value_dtype, const float *grad, float *gscale, float *gzp, cudaStream_t st);
size_t peer_flag_bytes();
size_t peer_state_bytes();
int peer_device_status();
int peer_allreduce_f16(const void *const *bufs, void *const *res, void *const *flags, int rank, int world, void *out, int64_t count,
                       void *state, cudaStream_t st);
int rtn_device_status();
long long div_self_check(unsigned long long n, unsigned long long seed);
int qmatmul_grad_input(const void *go, int dtype, int64_t M, int64_t N, int64_t K, const int32_t *q,
                       const __half *scale, const __half *zp, void *gi, int bits, int g, cudaStream_t st);

// Token counts above this go to the tensor-core GEMM, the rest to the streaming kernels.
static int64_t g_tc_min_tokens = 32;
#define TC_MIN_TOKENS g_tc_min_tokens

static bool is_float_dtype(int dt) { return dt == BW_F32 || dt == BW_F16 || dt == BW_BF16; }

}  // namespace bw

using namespace bw;

extern "C" {

int bw_rtn_quantize_pack(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int group_size,
                         int32_t *qweight, void *scale, int scale_dtype, void *zero_point,
                         int zp_dtype, unsigned flags, void *stream) {
    int rc = check_quant_shape(N, K, bits, group_size);
    if (rc != BW_OK) return rc;
    if (!is_float_dtype(w_dtype) || !is_float_dtype(scale_dtype)) return BW_ERR_DTYPE;
    if (zp_dtype != BW_I32 && zp_dtype != BW_F16) return BW_ERR_DTYPE;
    if (N * K == 0) return BW_OK;
    if (!w || !qweight || !scale || !zero_point) return BW_ERR_NULL;
    if (!aligned_to(w, dtype_size(w_dtype)) || !aligned_to(qweight, 4) ||
        !aligned_to(scale, dtype_size(scale_dtype)) || !aligned_to(zero_point, dtype_size(zp_dtype)))
        return BW_ERR_ALIGN;
    return rtn_quantize_pack(w, w_dtype, N, K, bits, group_size, qweight, scale, scale_dtype,
                             zero_point, zp_dtype, flags, (cudaStream_t)stream);
}

size_t bw_rtn_batch_table_bytes(int njobs) { return rtn_batch_table_bytes(njobs); }

int bw_rtn_quantize_pack_batch(const bw_rtn_job *jobs, int njobs, int w_dtype, int bits, int group_size,
                               int scale_dtype, int zp_dtype, unsigned flags, void *table_dev, size_t table_bytes,
                               void *stream) {
    if (njobs < 0) return BW_ERR_SHAPE;
    if (njobs == 0) return BW_OK;
    if (!jobs) return BW_ERR_NULL;
    if (!is_float_dtype(w_dtype) || !is_float_dtype(scale_dtype)) return BW_ERR_DTYPE;
    if (zp_dtype != BW_I32 && zp_dtype != BW_F16) return BW_ERR_DTYPE;
    for (int j = 0; j < njobs; ++j) {
        const bw_rtn_job &jb = jobs[j];
        const int rc = check_quant_shape(jb.N, jb.K, bits, group_size);
        if (rc != BW_OK) return rc;
        if (jb.N * jb.K == 0) continue;
        if (!jb.w || !jb.qweight || !jb.scale || !jb.zero_point) return BW_ERR_NULL;
        if (!aligned_to(jb.w, dtype_size(w_dtype)) || !aligned_to(jb.qweight, 4) ||
            !aligned_to(jb.scale, dtype_size(scale_dtype)) || !aligned_to(jb.zero_point, dtype_size(zp_dtype)))
            return BW_ERR_ALIGN;
    }
    if (table_dev && (table_bytes < rtn_batch_table_bytes(njobs) || !aligned_to(table_dev, 8))) return BW_ERR_WORKSPACE;
    return rtn_quantize_pack_batch(jobs, njobs, w_dtype, bits, group_size, scale_dtype, zp_dtype, flags, table_dev,
                                   (cudaStream_t)stream);
}

int bw_dequantize(const int32_t *qweight, const void *scale, int scale_dtype, const void *zero_point,
                  int zp_dtype, int64_t N, int64_t K, int bits, int group_size, void *out,
                  int out_dtype, void *stream) {
    int rc = check_quant_shape(N, K, bits, group_size);
    if (rc != BW_OK) return rc;
    if (!is_float_dtype(scale_dtype) || !is_float_dtype(out_dtype)) return BW_ERR_DTYPE;
    if (!is_float_dtype(zp_dtype) && zp_dtype != BW_I32) return BW_ERR_DTYPE;
    if (N * K == 0) return BW_OK;
    if (!qweight || !scale || !zero_point || !out) return BW_ERR_NULL;
    if (!aligned_to(qweight, 4) || !aligned_to(scale, dtype_size(scale_dtype)) ||
        !aligned_to(zero_point, dtype_size(zp_dtype)) || !aligned_to(out, dtype_size(out_dtype)))
        return BW_ERR_ALIGN;
    return dequantize(qweight, scale, scale_dtype, zero_point, zp_dtype, N, K, bits, group_size, out,
                      out_dtype, (cudaStream_t)stream);
}

// Scratch of the cluster split-K streaming kernel and the tensor-core GEMM (everything that
// bw_qmatmul_noalloc can run).  The streaming kernel reads activations that a preparation
// kernel has cast to fp16 and laid out in tensor-core fragment order: K (rounded up to a
// k-chunk) x 8*ceil(M/8) x 2 bytes for one block of at most 64 tokens; its split-K sums travel
// through distributed shared memory and need no global scratch.
static size_t cluster_path_workspace_bytes(int64_t M, int64_t K, int bits) {
    if (bits != 2 && bits != 4 && bits != 8) return 0;
    if (M <= 0 || K <= 0) return 0;
    const size_t small = smallm_workspace_bytes(M < 64 ? M : 64, K, bits);
    if (M <= TC_MIN_TOKENS) return small;
    // the tensor-core kernel reads fp16 activations; other dtypes are cast into the workspace
    const size_t cast = tc_workspace_bytes(M, K);
    return cast > small ? cast : small;
}

size_t bw_qmatmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int bits, int group_size) {
    (void)group_size;
    const size_t base = cluster_path_workspace_bytes(M, K, bits);
    if (base == 0 || M > 32 || N <= 0) return base;
    // the persistent decode kernel adds row-block counters and stream-K partial tiles
    const size_t dec = decode_workspace_bytes(M, N, K, bits);
    return dec > base ? dec : base;
}

size_t bw_qmatmul_workspace_bytes_for(int64_t M, int64_t N, int64_t K, int bits, int group_size, int x_dtype, int x_align) {
    const size_t all = bw_qmatmul_workspace_bytes(M, N, K, bits, group_size);
    if (M <= TC_MIN_TOKENS || x_dtype != BW_F16 || x_align < 16) return all;
    // more than 32 tokens of aligned fp16: the GEMM reads them in place; only layouts the GEMM
    // cannot take need the streaming kernel's prepared activations
    const size_t small = smallm_workspace_bytes(64, K, bits);
    return small < all ? small : all;
}

// Argument checks shared by the qmatmul entry points (before any CUDA call).
static int qmatmul_validate(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *qweight,
                            const void *scale, const void *zero_point, const void *bias, void *out, int out_dtype,
                            int bits, int group_size) {
    int rc = check_quant_shape(N, K, bits, group_size);
    if (rc != BW_OK) return rc;
    if (M < 0) return BW_ERR_SHAPE;
    if (!is_float_dtype(x_dtype) || !is_float_dtype(out_dtype)) return BW_ERR_DTYPE;
    if (M == 0 || N == 0) return BW_OK;
    if (!out) return BW_ERR_NULL;
    if (K > 0 && (!x || !qweight || !scale || !zero_point)) return BW_ERR_NULL;
    if (!aligned_to(x, dtype_size(x_dtype)) || !aligned_to(out, dtype_size(out_dtype)) ||
        !aligned_to(qweight, 4) || !aligned_to(scale, 2) || !aligned_to(zero_point, 2) ||
        !aligned_to(bias, 2))
        return BW_ERR_ALIGN;
    return BW_OK;
}

// `persistent_decode`: let M <= 32 run on the persistent TMA-fed decode kernel (needs the larger
// workspace of bw_qmatmul_workspace_bytes); otherwise only the cluster split-K streaming kernel
// and the tensor-core GEMM are used.  `allow_tc`: the tensor-core GEMM may be used (its
// activation cast, where one is needed, fits the workspace).
static int qmatmul_dispatch(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *qweight,
                            const void *scale, const void *zero_point, const void *bias, void *out, int out_dtype,
                            int bits, int group_size, void *workspace, size_t workspace_bytes, void *stream,
                            bool persistent_decode, bool allow_tc) {
    int rc = qmatmul_validate(x, x_dtype, M, N, K, qweight, scale, zero_point, bias, out, out_dtype, bits, group_size);
    if (rc != BW_OK) return rc;
    if (M == 0 || N == 0) return BW_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const __half *s = (const __half *)scale, *z = (const __half *)zero_point, *b = (const __half *)bias;
    // the gated epilogue pairs adjacent weight rows: only the decode and tensor-core kernels do that
    const bool paired = g_epilogue.act == BW_ACT_SILU_MUL;
    if (paired && (K == 0 || !smallm_fast_path_ok(x, x_dtype, K, qweight, bits, group_size))) return BW_ERR_UNSUPPORTED;
    if (K == 0) {
        // empty reduction: out = bias (or 0); run the general kernel, which handles it
        return qmatmul_smallm(x, x_dtype, M, N, K, qweight, s, z, b, out, out_dtype, bits, group_size, nullptr, st);
    }
    if (!smallm_fast_path_ok(x, x_dtype, K, qweight, bits, group_size))
        return qmatmul_smallm(x, x_dtype, M, N, K, qweight, s, z, b, out, out_dtype, bits, group_size, nullptr, st);
    if (persistent_decode && M <= 32 && decode_path_ok(x, x_dtype, M, N, K, qweight, scale, zero_point, bits, group_size)) {
        if (!workspace || workspace_bytes < bw_qmatmul_workspace_bytes(M, N, K, bits, group_size))
            return BW_ERR_WORKSPACE;
        rc = qmatmul_decode(x, x_dtype, M, N, K, qweight, s, z, b, out, out_dtype, bits, group_size, workspace, st);
        if (rc != BW_ERR_UNSUPPORTED || paired) return rc;   // otherwise nothing was launched: use the cluster split-K kernel
    }
    if (allow_tc && M > TC_MIN_TOKENS && tc_path_ok(M, N, K, qweight, bits, group_size)) {
        const bool direct = x_dtype == BW_F16 && aligned_to(x, 16);   // TMA reads fp16 activations as they are
        if (!direct && (!workspace || workspace_bytes < tc_workspace_bytes(M, K))) return BW_ERR_WORKSPACE;
        return qmatmul_tc(x, x_dtype, M, N, K, qweight, s, z, b, out, out_dtype, bits, group_size, workspace, st);
    }
    if (paired) return BW_ERR_UNSUPPORTED;
    // token blocks of at most 64 through the streaming kernel
    if (!workspace || workspace_bytes < smallm_workspace_bytes(M < 64 ? M : 64, K, bits)) return BW_ERR_WORKSPACE;
    const size_t xs = dtype_size(x_dtype), os = dtype_size(out_dtype);
    for (int64_t m0 = 0; m0 < M; m0 += 64) {
        const int64_t mc = (M - m0 < 64) ? (M - m0) : 64;
        rc = qmatmul_smallm((const char *)x + (size_t)m0 * K * xs, x_dtype, mc, N, K, qweight, s, z, b,
                            (char *)out + (size_t)m0 * N * os, out_dtype, bits, group_size, workspace, st);
        if (rc != BW_OK) return rc;
    }
    return BW_OK;
}

int bw_qmatmul(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *qweight,
               const void *scale, const void *zero_point, const void *bias, void *out, int out_dtype,
               int bits, int group_size, void *workspace, size_t workspace_bytes, void *stream) {
    return qmatmul_dispatch(x, x_dtype, M, N, K, qweight, scale, zero_point, bias, out, out_dtype, bits,
                            group_size, workspace, workspace_bytes, stream, true, true);
}

int bw_qmatmul_fused(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K, const int32_t *qweight,
                     const void *scale, const void *zero_point, const void *bias, void *out, int out_dtype,
                     int bits, int group_size, const bw_epilogue *ep, void *workspace, size_t workspace_bytes,
                     void *stream) {
    if (ep) {
        if (ep->activation != BW_ACT_NONE && ep->activation != BW_ACT_RELU && ep->activation != BW_ACT_SILU_MUL) return BW_ERR_UNSUPPORTED;
        if (ep->activation == BW_ACT_SILU_MUL && N % 4 != 0) return BW_ERR_SHAPE;
        if (!aligned_to(ep->residual, 2)) return BW_ERR_ALIGN;
        g_epilogue = {ep->activation, reinterpret_cast<const __half *>(ep->residual)};
    }
    const int rc = qmatmul_dispatch(x, x_dtype, M, N, K, qweight, scale, zero_point, bias, out, out_dtype, bits,
                                    group_size, workspace, workspace_bytes, stream, true, true);
    g_epilogue = {BW_ACT_NONE, nullptr};
    return rc;
}

int bw_qmatmul_noalloc(const void *x, int x_dtype, int64_t M, int64_t N, int64_t K,
                       const int32_t *qweight, const void *scale, const void *zero_point,
                       const void *bias, void *out, int out_dtype, int bits, int group_size,
                       void *stream) {
    int rc = qmatmul_validate(x, x_dtype, M, N, K, qweight, scale, zero_point, bias, out, out_dtype, bits, group_size);
    if (rc != BW_OK) return rc;
    if (M == 0 || N == 0) return BW_OK;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    rc = noalloc_scratch(&scratch, &scratch_bytes);
    if (rc != BW_OK) return rc;
    // What the kernel that will run really needs from the built-in scratch: nothing for the
    // general kernel and for the tensor-core GEMM on 16-byte-aligned fp16 activations; M*K*2 bytes
    // for the GEMM's fp16 cast of other activations -- when that does not fit, token blocks of 64
    // go through the streaming kernel instead; the streaming kernel's prepared activations
    // (K rounded up to a k-chunk x 8*ceil(min(M,64)/8) x 2 bytes) otherwise.  Requests that do not
    // fit are refused before anything is launched.
    bool allow_tc = true;
    size_t need = 0;
    if (K > 0 && smallm_fast_path_ok(x, x_dtype, K, qweight, bits, group_size)) {
        const bool tc = M > TC_MIN_TOKENS && tc_path_ok(M, N, K, qweight, bits, group_size);
        const bool direct = x_dtype == BW_F16 && aligned_to(x, 16);
        if (tc && direct) need = 0;
        else if (tc && tc_workspace_bytes(M, K) <= scratch_bytes) need = tc_workspace_bytes(M, K);
        else {
            allow_tc = false;
            need = smallm_workspace_bytes(M < 64 ? M : 64, K, bits);
        }
    }
    if (need > scratch_bytes) return BW_ERR_TOO_LARGE;
    return qmatmul_dispatch(x, x_dtype, M, N, K, qweight, scale, zero_point, bias, out, out_dtype, bits,
                            group_size, scratch, scratch_bytes, stream, false, allow_tc);
}

size_t bw_qmatmul_noalloc_max_scratch_bytes(void) {
    void *p = nullptr;
    size_t b = 0;
    return noalloc_scratch(&p, &b) == BW_OK ? b : 0;
}

// Staging between pinned host memory and the device for bw_qmatmul_host.  Decode-sized
// activations and outputs are a few KB to a few hundred KB: a copy engine needs several
// microseconds of set-up per transfer and serialises with the kernel, so they are moved by a
// small kernel instead -- plain 16-byte loads / stores on the host buffer's device mapping
// (pinned memory is mapped into the unified address space), launched with programmatic
// stream serialisation so that its launch latency overlaps its predecessor.
__global__ void __launch_bounds__(256) staging_copy_kernel(const unsigned char *__restrict__ src,
                                                           unsigned char *__restrict__ dst, size_t bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");      // dst may still be read, src still be written, by the predecessor
    const size_t n16 = bytes / 16;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < n16; i += stride)
        reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
    for (size_t i = n16 * 16 + tid; i < bytes; i += stride) dst[i] = src[i];
}

// The device-side address of a pinned (mapped) host buffer, or nullptr.
static void *device_view_of_host(const void *host) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

static constexpr size_t STAGING_KERNEL_MAX_BYTES = (size_t)4 << 20;   // larger transfers go to the copy engines

static int staging_copy(void *dst, const void *src, size_t bytes, cudaMemcpyKind kind, cudaStream_t st) {
    if (bytes == 0) return BW_OK;
    const void *host = kind == cudaMemcpyHostToDevice ? src : dst;
    void *mapped = bytes <= STAGING_KERNEL_MAX_BYTES && aligned_to(dst, 16) && aligned_to(src, 16) ? device_view_of_host(host) : nullptr;
    if (!mapped) {
        BW_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, kind, st));
        return BW_OK;
    }
    const void *s = kind == cudaMemcpyHostToDevice ? mapped : src;
    void *d = kind == cudaMemcpyHostToDevice ? dst : mapped;
    size_t blocks = (bytes / 16 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 64) blocks = 64;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BW_CUDA_TRY(cudaLaunchKernelEx(&cfg, staging_copy_kernel, (const unsigned char *)s, (unsigned char *)d, bytes));
    return BW_OK;
}

int bw_qmatmul_host(const void *x_host, int x_dtype, int64_t M, int64_t N, int64_t K,
                    const int32_t *qweight, const void *scale, const void *zero_point,
                    const void *bias, void *out_host, int out_dtype, int bits, int group_size,
                    void *x_dev, void *out_dev, void *workspace, size_t workspace_bytes,
                    void *stream) {
    if (M < 0 || N < 0 || K < 0) return BW_ERR_SHAPE;
    if (!is_float_dtype(x_dtype) || !is_float_dtype(out_dtype)) return BW_ERR_DTYPE;
    if (M * N == 0) return BW_OK;
    if (!x_dev || !out_dev || !out_host || (K > 0 && !x_host)) return BW_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = staging_copy(x_dev, x_host, (size_t)(M * K) * dtype_size(x_dtype), cudaMemcpyHostToDevice, st);
    if (rc != BW_OK) return rc;
    rc = bw_qmatmul(x_dev, x_dtype, M, N, K, qweight, scale, zero_point, bias, out_dev, out_dtype,
                    bits, group_size, workspace, workspace_bytes, stream);
    if (rc != BW_OK) return rc;
    return staging_copy(out_host, out_dev, (size_t)(M * N) * dtype_size(out_dtype), cudaMemcpyDeviceToHost, st);
}

int bw_qmatmul_grad_input(const void *grad_out, int grad_dtype, int64_t M, int64_t N, int64_t K,
                          const int32_t *qweight, const void *scale, const void *zero_point,
                          void *grad_in, int bits, int group_size, void *stream) {
    int rc = check_quant_shape(N, K, bits, group_size);
    if (rc != BW_OK) return rc;
    if (M < 0) return BW_ERR_SHAPE;
    if (!is_float_dtype(grad_dtype)) return BW_ERR_DTYPE;
    if (M == 0 || K == 0) return BW_OK;
    if (!grad_in) return BW_ERR_NULL;
    if (N > 0 && (!grad_out || !qweight || !scale || !zero_point)) return BW_ERR_NULL;
    if (!aligned_to(grad_out, dtype_size(grad_dtype)) || !aligned_to(grad_in, dtype_size(grad_dtype)) ||
        !aligned_to(qweight, 4) || !aligned_to(scale, 2) || !aligned_to(zero_point, 2))
        return BW_ERR_ALIGN;
    return qmatmul_grad_input(grad_out, grad_dtype, M, N, K, qweight, (const __half *)scale,
                              (const __half *)zero_point, grad_in, bits, group_size,
                              (cudaStream_t)stream);
}

int bw_fake_quant(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int group_size, const float *scale,
                  const float *zero_point, const void *value, int value_dtype, float *w_dq, float *w_q, void *stream) {
    if (bits != 2 && bits != 4 && bits != 8) return BW_ERR_BITS;
    if (group_size < 1) return BW_ERR_GROUP;
    if (N < 0 || K < 0) return BW_ERR_SHAPE;
    if (K % group_size != 0) return BW_ERR_GROUP;
    if (!is_float_dtype(w_dtype) || (value && !is_float_dtype(value_dtype))) return BW_ERR_DTYPE;
    if (N * K == 0) return BW_OK;
    if (!w || !scale || !zero_point || !w_dq) return BW_ERR_NULL;
    if (!aligned_to(w, dtype_size(w_dtype)) || !aligned_to(scale, 4) || !aligned_to(zero_point, 4) ||
        (value && !aligned_to(value, dtype_size(value_dtype))) ||
        !aligned_to(w_dq, 4) || !aligned_to(w_q, 4))
        return BW_ERR_ALIGN;
    return fake_quant(w, w_dtype, N, K, bits, group_size, scale, zero_point, value, value_dtype, w_dq, w_q, (cudaStream_t)stream);
}

int bw_fake_quant_native16(const void *w, int dtype, int64_t N, int64_t K, int bits, int group_size, const void *scale,
                           const void *zero_point, const void *value, void *w_dq, void *w_q, void *stream) {
    if (bits != 2 && bits != 4 && bits != 8) return BW_ERR_BITS;
    if (group_size < 1) return BW_ERR_GROUP;
    if (N < 0 || K < 0) return BW_ERR_SHAPE;
    if (K % group_size != 0) return BW_ERR_GROUP;
    if (dtype != BW_F16 && dtype != BW_BF16) return BW_ERR_DTYPE;
    if (N * K == 0) return BW_OK;
    if (!w || !scale || !zero_point || !w_dq) return BW_ERR_NULL;
    if (!aligned_to(w, 2) || !aligned_to(scale, 2) || !aligned_to(zero_point, 2) || !aligned_to(value, 2) || !aligned_to(w_dq, 2) ||
        !aligned_to(w_q, 2))
        return BW_ERR_ALIGN;
    return fake_quant_native(w, dtype, N, K, bits, group_size, scale, zero_point, value, w_dq, w_q, (cudaStream_t)stream);
}

int bw_fake_quant_backward(const void *w, int w_dtype, int64_t N, int64_t K, int bits, int group_size, const float *scale,
                           const float *zero_point, const void *value, int value_dtype, const float *grad_w_dq,
                           float *grad_scale, float *grad_zero_point, void *stream) {
    if (bits != 2 && bits != 4 && bits != 8) return BW_ERR_BITS;
    if (group_size < 1) return BW_ERR_GROUP;
    if (N < 0 || K < 0) return BW_ERR_SHAPE;
    if (K % group_size != 0) return BW_ERR_GROUP;
    if (!is_float_dtype(w_dtype) || (value && !is_float_dtype(value_dtype))) return BW_ERR_DTYPE;
    if (N * K == 0) return BW_OK;
    if (!w || !scale || !zero_point || !grad_w_dq || !grad_scale || !grad_zero_point) return BW_ERR_NULL;
    if (!aligned_to(scale, 4) || !aligned_to(zero_point, 4) || !aligned_to(grad_scale, 4) || !aligned_to(grad_zero_point, 4))
        return BW_ERR_ALIGN;
    return fake_quant_backward(w, w_dtype, N, K, bits, group_size, scale, zero_point, value, value_dtype, grad_w_dq, grad_scale,
                               grad_zero_point, (cudaStream_t)stream);
}

// ---- peer-memory all-reduce (row-parallel layers on one node) ----
int bw_peer_alloc(size_t bytes, void **ptr, unsigned char *ipc_handle) {
    if (!ptr || !ipc_handle || bytes == 0) return BW_ERR_NULL;
    void *p = nullptr;
    BW_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        (void)cudaFree(p);
        return record_cuda_error(e, "bw_peer_alloc");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(ipc_handle, &h, sizeof(h));
    *ptr = p;
    return BW_OK;
}
int bw_peer_open(const unsigned char *ipc_handle, void **ptr) {
    if (!ptr || !ipc_handle) return BW_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    BW_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return BW_OK;
}
int bw_peer_close(void *ptr) {
    if (!ptr) return BW_OK;
    BW_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return BW_OK;
}
int bw_peer_free(void *ptr) {
    if (!ptr) return BW_OK;
    BW_CUDA_TRY(cudaFree(ptr));
    return BW_OK;
}
size_t bw_peer_flag_bytes(void) { return peer_flag_bytes(); }
size_t bw_peer_state_bytes(void) { return peer_state_bytes(); }
int bw_peer_allreduce_f16(const void *const *bufs, void *const *flags, int rank, int world, void *out, int64_t count,
                          void *state, void *stream) {
    return peer_allreduce_f16(bufs, nullptr, flags, rank, world, out, count, state, (cudaStream_t)stream);
}
int bw_peer_allreduce2_f16(const void *const *bufs, void *const *results, void *const *flags, int rank, int world, void *out,
                           int64_t count, void *state, void *stream) {
    if (!results) return BW_ERR_NULL;
    return peer_allreduce_f16(bufs, results, flags, rank, world, out, count, state, (cudaStream_t)stream);
}

const char *bw_status_string(int status) {
    switch (status) {
        case BW_OK: return "ok";
        case BW_ERR_BITS: return "Only 2, 4, or 8-bit quantization supported.";
        case BW_ERR_GROUP: return "group_size must be >= 1 and divide in_features";
        case BW_ERR_SHAPE: return "bad shape (negative, too large, or in_features not a multiple of 32/bits)";
        case BW_ERR_DTYPE: return "dtype not accepted for this argument";
        case BW_ERR_ALIGN: return "pointer not aligned for its element type";
        case BW_ERR_NULL: return "required pointer is NULL";
        case BW_ERR_WORKSPACE: return "workspace too small";
        case BW_ERR_CUDA: return "CUDA runtime error (see bw_last_cuda_error)";
        case BW_ERR_UNSUPPORTED: return "no kernel for this request";
        case BW_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case BW_ERR_TOO_LARGE:
            return "request needs more scratch than the 2 MiB built into bw_qmatmul_noalloc "
                   "(prepared activations of the streaming kernel: K rounded up to a k-chunk x 8*ceil(min(M,64)/8) x 2 bytes); "
                   "use bw_qmatmul with a workspace";
        default: return "unknown status";
    }
}

const char *bw_last_cuda_error(void) { return g_cuda_error; }

int bw_device_status(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return record_cuda_error(cudaGetLastError(), "cudaDeviceSynchronize");
    const int v = rtn_device_status(), t = tc_device_status(), d = decode_device_status(), pr = peer_device_status();
    if (v < 0 || t < 0 || d < 0 || pr < 0) return BW_ERR_CUDA;
    return (v || t || d || pr) ? BW_ERR_TIMEOUT : BW_OK;
}
int bw_version(void) { return 100; }
const char *bw_last_qmatmul_kernel(void) { return g_last_kernel; }

#ifdef BW_TUNING
// Tuning build only (-DBW_TUNING): process-wide, unsynchronised switches for kernel experiments.
BW_API void bw_debug_set_smallm_tuning(int rt, int warps, int splits) { set_smallm_tuning(rt, warps, splits); }
BW_API void bw_debug_set_pdl(int on) { set_smallm_pdl(on); }
BW_API void bw_debug_set_decode(int enabled, int smem_kb, int max_ctas, int pdl) { set_decode_tuning(enabled, smem_kb, max_ctas, pdl); }
BW_API void bw_debug_set_tc(int on) { set_tc_enabled(on); }
BW_API void bw_debug_set_tc_splits(int s) { set_tc_splits(s); }
BW_API void bw_debug_set_tc_min_tokens(int m) { g_tc_min_tokens = m; }
#endif
long long bw_selftest_division(unsigned long long n, unsigned long long seed) { return div_self_check(n, seed); }

}  // extern "C"
