// Dynamic Tanh, a norm without statistics:  y = tanh(alpha * s) * w + b  with one learned scalar alpha and
// learned vectors w and b.  Every element stands alone, so the kernel is a plain elementwise pass; what it
// fuses is the residual arithmetic around it:
//
//   br  = branch                                  (absent: no branch)
//   br  = tanh(b_alpha * br) * b_w + b_b          (only if the branch has a Dynamic Tanh of its own: a block
//                                                  that norms a sublayer's output before adding it)
//   s   = x[src] + branch_scale * br              src = rows[r] (a row gather) or r
//   sum_out[r] = s                                (nullable; may be x itself when no rows are gathered)
//   out[r]     = tanh(alpha * s) * w + b          (nullable: only the sum is wanted)
//
// All arithmetic is float32 whatever the storage types are: x and sum_out share TX (the residual stream),
// the branch has TB, the normed row TO.
#include "common.cuh"

template <typename TX, typename TB, typename TO>
__global__ void dyt_kernel(TO* __restrict__ out, TX* sum_out, const TX* x, const TB* __restrict__ branch,
                           const int* __restrict__ rows, const float* __restrict__ alpha, const float* __restrict__ w,
                           const float* __restrict__ b, float branch_scale, const float* __restrict__ b_alpha,
                           const float* __restrict__ b_w, const float* __restrict__ b_b, int nrows, int dim, int src_rows,
                           int* err) {
    const float a = out ? alpha[0] : 0.f;
    const float ba = b_alpha ? b_alpha[0] : 0.f;
    for (int r = blockIdx.y; r < nrows; r += gridDim.y) {
        int src = rows ? rows[r] : r;
        if (src < 0 || src >= src_rows) {
            if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
            src = 0;
        }
        const TX* xr = x + (size_t)src * dim;
        const TB* br = branch ? branch + (size_t)src * dim : nullptr;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x) {
            float s = to_f32<TX>(xr[i]);
            if (br) {
                float v = to_f32<TB>(br[i]);
                if (b_alpha) v = fmaf(tanhf(ba * v), b_w[i], b_b[i]);
                s = fmaf(branch_scale, v, s);
            }
            if (sum_out) sum_out[(size_t)r * dim + i] = from_f32<TX>(s);
            if (out) out[(size_t)r * dim + i] = from_f32<TO>(fmaf(tanhf(a * s), w[i], b[i]));
        }
    }
}

template <typename TX, typename TB, typename TO>
static int dyt_launch(void* out, void* sum_out, const void* x, const void* branch, const int* rows, const float* alpha,
                      const float* w, const float* b, float branch_scale, const float* b_alpha, const float* b_w,
                      const float* b_b, int nrows, int dim, int src_rows, int* err, cudaStream_t stream) {
    const int threads = dim >= 1024 ? 256 : 128;
    int bx = (dim + threads * 4 - 1) / (threads * 4);
    if (bx < 1) bx = 1;
    dyt_kernel<TX, TB, TO><<<dim3(bx, nrows < 65535 ? nrows : 65535), threads, 0, stream>>>((TO*)out, (TX*)sum_out, (const TX*)x, (const TB*)branch, rows,
                                                                     alpha, w, b, branch_scale, b_alpha, b_w, b_b, nrows, dim,
                                                                     src_rows, err);
    return xb_launch_status();
}

XB_EXPORT int xb_dyt_norm(int x_dtype, int branch_dtype, int out_dtype, void* out, void* sum_out, const void* x,
                          const void* branch, const int* rows, const float* alpha, const float* w, const float* b,
                          float branch_scale, const float* b_alpha, const float* b_w, const float* b_b, int nrows, int dim,
                          int src_rows, int* err, cudaStream_t stream) {
    if (nrows <= 0 || dim <= 0) return 0;
    typedef __nv_bfloat16 bf;
#define XB_ARGS out, sum_out, x, branch, rows, alpha, w, b, branch_scale, b_alpha, b_w, b_b, nrows, dim, src_rows, err, stream
#define XB_PICK_O(TX, TB) (out_dtype == XB_F32 ? dyt_launch<TX, TB, float>(XB_ARGS) : dyt_launch<TX, TB, bf>(XB_ARGS))
#define XB_PICK_B(TX) (branch_dtype == XB_F32 ? XB_PICK_O(TX, float) : XB_PICK_O(TX, bf))
    return x_dtype == XB_F32 ? XB_PICK_B(float) : XB_PICK_B(bf);
#undef XB_PICK_B
#undef XB_PICK_O
#undef XB_ARGS
}
