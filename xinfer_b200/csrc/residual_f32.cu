// Kernels for models whose residual stream is float32 while the engine's matrix products run in
// bfloat16: the embedding gather that widens its rows, the norm that reads the float32 stream (plus
// a branch in either type), stores the float32 sum and writes the normed row in the engine's type,
// and the addition of a branch into the stream.  Sums and statistics are float32; a row is reduced
// in an order fixed by the thread layout, so a row's result does not depend on the batch.
#include "common.cuh"

template <typename T>
__global__ void embedding_f32_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                     const int* __restrict__ sampled, int num_sampled, int hidden, int vocab, float scale,
                                     int* err) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && sampled != nullptr && -1 - id < num_sampled) id = sampled[-1 - id];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* r = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32<T>(r[i]) * scale;
}

XB_EXPORT int xb_embedding_f32(int table_dtype, float* out, const void* table, const int* ids, const int* sampled,
                               int num_sampled, int tokens, int hidden, int vocab, float scale, int* err,
                               cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (table_dtype == XB_F32)
        embedding_f32_kernel<float><<<tokens, 256, 0, stream>>>(out, (const float*)table, ids, sampled, num_sampled, hidden, vocab, scale, err);
    else
        embedding_f32_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(out, (const __nv_bfloat16*)table, ids, sampled, num_sampled, hidden, vocab, scale, err);
    return xb_launch_status();
}

//   s   = x[src] (+ branch[src])               float32
//   out = s * rsqrt(mean(s^2) + eps) * (offset + w)     in TO
// sum_out (float32, nullable) receives s; it may be x itself when no rows are gathered.
template <typename TB, typename TO>
__global__ void rmsnorm_f32_kernel(TO* __restrict__ out, float* sum_out, const float* x, const TB* __restrict__ branch,
                                   const int* __restrict__ rows, const float* __restrict__ w, int dim, int src_rows,
                                   float eps, float offset, int* err) {
    __shared__ float scratch[33];
    extern __shared__ float srow[];
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= src_rows) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
        src = 0;
    }
    const float* xr = x + (size_t)src * dim;
    const TB* br = branch ? branch + (size_t)src * dim : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = xr[i];
        if (br) v += to_f32<TB>(br[i]);
        srow[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(total / (float)dim + eps);
    TO* o = out + (size_t)r * dim;
    float* so = sum_out ? sum_out + (size_t)r * dim : nullptr;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = srow[i];
        if (so) so[i] = v;
        o[i] = from_f32<TO>(v * inv * (offset + w[i]));
    }
}

template <typename TB, typename TO>
static int rmsnorm_f32_launch(void* out, float* sum_out, const float* x, const void* branch, const int* rows, const float* w,
                              int nrows, int dim, int src_rows, float eps, float offset, int* err, cudaStream_t stream) {
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_f32_kernel<TB, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    rmsnorm_f32_kernel<TB, TO><<<nrows, threads, smem, stream>>>((TO*)out, sum_out, x, (const TB*)branch, rows, w, dim, src_rows,
                                                                eps, offset, err);
    return xb_launch_status();
}

XB_EXPORT int xb_rmsnorm_f32(int branch_dtype, int out_dtype, void* out, float* sum_out, const float* x, const void* branch,
                             const int* rows, const float* w, int nrows, int dim, int src_rows, float eps, float offset,
                             int* err, cudaStream_t stream) {
    if (nrows <= 0) return 0;
    typedef __nv_bfloat16 bf;
#define XB_ARGS out, sum_out, x, branch, rows, w, nrows, dim, src_rows, eps, offset, err, stream
    if (branch_dtype == XB_F32) return out_dtype == XB_F32 ? rmsnorm_f32_launch<float, float>(XB_ARGS) : rmsnorm_f32_launch<float, bf>(XB_ARGS);
    return out_dtype == XB_F32 ? rmsnorm_f32_launch<bf, float>(XB_ARGS) : rmsnorm_f32_launch<bf, bf>(XB_ARGS);
#undef XB_ARGS
}

template <typename TB>
__global__ void add_f32_kernel(float* out, const float* x, const TB* branch, size_t n, float scale) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = scale == 1.f ? x[i] + to_f32<TB>(branch[i]) : fmaf(scale, to_f32<TB>(branch[i]), x[i]);
}

XB_EXPORT int xb_add_f32(int branch_dtype, float* out, const float* x, const void* branch, long long n, float scale, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (branch_dtype == XB_F32)
        add_f32_kernel<float><<<blocks, 256, 0, stream>>>(out, x, (const float*)branch, (size_t)n, scale);
    else
        add_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(out, x, (const __nv_bfloat16*)branch, (size_t)n, scale);
    return xb_launch_status();
}
