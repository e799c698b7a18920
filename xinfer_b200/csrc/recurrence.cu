// Gated recurrence whose gates read only the current token (minGRU), and the polynomial activation
// that norms each power.  Everything here is float32 arithmetic; inputs are the float32 outputs
// of the projections.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
//   zxg[t] = [W_z h | W_x h | W_g h]  (3 x width, float32, biases not yet added)
//   z = sigmoid(zxg_z + bz),  u = zxg_x + bx,  c = u >= 0 ? u + 1/2 : sigmoid(u)
//   S <- (1 - z) S + z c          per channel; S of an entry lives in state[slot] between steps
//   y[t] = out_scale * S * silu(zxg_g)
// A step's tokens of one entry are consecutive rows, in order.  Two forms:
//  * serial: a thread per (entry, channel) walks over the entry's tokens;
//  * chunked, for long portions: the recurrence S_t = a_t S_(t-1) + b_t is cut into chunks of CH
//    tokens; pass 1 gives each chunk its product of a and its own end value from zero, pass 2 walks
//    over an entry's chunks to give each its start value, pass 3 redoes each chunk from that start
//    and writes y.  The additions happen in the same order as in the serial form inside a chunk,
//    and differ across chunk borders only by rounding.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoid_f32(float v) { return 1.f / (1.f + expf(-v)); }

__device__ __forceinline__ void gate_and_candidate(const float* __restrict__ row, int W, int c, float bz, float bx,
                                                   float& a, float& b) {
    const float z = sigmoid_f32(row[c] + bz);
    const float u = row[W + c] + bx;
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f32(u);
    a = 1.f - z;
    b = z * cand;
}

template <typename T>
__global__ void gated_scan_serial_kernel(T* __restrict__ y, int ldy, const float* __restrict__ zxg,
                                         const float* __restrict__ bz, const float* __restrict__ bx,
                                         float* __restrict__ state, const int* __restrict__ q_start,
                                         const int* __restrict__ slots, int W, float out_scale) {
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = slots[b];
    if (c >= W || slot < 0) return;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    float S = state[(size_t)slot * W + c];
    const float vz = bz[c], vx = bx[c];
    for (int t = t0; t < t1; ++t) {
        const float* row = zxg + (size_t)t * 3 * W;
        float a, bb;
        gate_and_candidate(row, W, c, vz, vx, a, bb);
        S = fmaf(a, S, bb);
        const float g = row[2 * W + c];
        y[(size_t)t * ldy + c] = from_f32<T>(S * (g * sigmoid_f32(g)) * out_scale);
    }
    state[(size_t)slot * W + c] = S;
}

// chunked form.  Chunks are counted over the step's rows: chunk k covers rows [k*CH, (k+1)*CH); a chunk
// that crosses an entry's border is handled per entry by restarting at the border (req_of_token tells).
constexpr int GS_CH = 32;

// pass 1: per (chunk, channel), for every entry piece inside the chunk: A = prod a, Bv = value from zero.
// A chunk holds at most a few pieces; to keep it simple a piece is identified by its first row, and
// results are stored per row range as "value and product up to the end of the row's piece within the
// chunk" at the piece's last row.
__global__ void gated_scan_chunk_kernel(float* __restrict__ prodA, float* __restrict__ endB,
                                        const float* __restrict__ zxg, const float* __restrict__ bz,
                                        const float* __restrict__ bx, const int* __restrict__ req_of_token, int T, int W) {
    const int k = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int r0 = k * GS_CH, r1 = min(T, r0 + GS_CH);
    const float vz = bz[c], vx = bx[c];
    float A = 1.f, B = 0.f;
    int cur = r0 < T ? req_of_token[r0] : -1;
    for (int t = r0; t < r1; ++t) {
        const int rq = req_of_token[t];
        if (rq != cur) { A = 1.f; B = 0.f; cur = rq; }      // a new entry starts inside the chunk
        float a, bb;
        gate_and_candidate(zxg + (size_t)t * 3 * W, W, c, vz, vx, a, bb);
        A *= a;
        B = fmaf(a, B, bb);
        // the running pair of the piece that row t belongs to, up to and including t
        prodA[(size_t)t * W + c] = A;
        endB[(size_t)t * W + c] = B;
    }
}

// pass 2 + 3: per (entry, channel) walk over the entry's chunk ends to find each chunk's start value, then
// every row's state is  S_t = prodA[t] * start(piece of t) + endB[t]; one thread per (row, channel) would
// need the start values, so they are kept per chunk piece in `start` ([rows, W] at the piece's first row).
__global__ void gated_scan_starts_kernel(float* __restrict__ start, const float* __restrict__ prodA,
                                         const float* __restrict__ endB, float* __restrict__ state,
                                         const int* __restrict__ q_start, const int* __restrict__ slots, int W) {
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = slots[b];
    if (c >= W || slot < 0) return;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    float S = state[(size_t)slot * W + c];
    // pieces: [t0, first chunk border), then whole chunks, then the rest; four pieces' pairs are loaded ahead
    // of the recurrence, which only needs them one after the other
    int t = t0;
    while (t < t1) {
        int first[4], last[4];
        float A[4], B[4];
        int n = 0;
        for (int tt = t; n < 4 && tt < t1; ++n) {
            first[n] = tt;
            tt = min(t1, (tt / GS_CH + 1) * GS_CH);
            last[n] = tt - 1;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (k < n) {
                A[k] = prodA[(size_t)last[k] * W + c];
                B[k] = endB[(size_t)last[k] * W + c];
            }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (k < n) {
                start[(size_t)first[k] * W + c] = S;
                S = fmaf(A[k], S, B[k]);
            }
        t = last[n - 1] + 1;
    }
    state[(size_t)slot * W + c] = S;
}

template <typename T>
__global__ void gated_scan_finish_kernel(T* __restrict__ y, int ldy, const float* __restrict__ zxg,
                                         const float* __restrict__ start, const float* __restrict__ prodA,
                                         const float* __restrict__ endB, const int* __restrict__ req_of_token,
                                         const int* __restrict__ q_start, int tokens, int W, float out_scale) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W || t >= tokens) return;
    const int b = req_of_token[t];
    if (b < 0) return;
    // first row of the piece that t belongs to: the chunk's first row or the entry's first row
    const int first = max(t / GS_CH * GS_CH, q_start[b]);
    const float S = fmaf(prodA[(size_t)t * W + c], start[(size_t)first * W + c], endB[(size_t)t * W + c]);
    const float g = zxg[(size_t)t * 3 * W + 2 * W + c];
    y[(size_t)t * ldy + c] = from_f32<T>(S * (g * sigmoid_f32(g)) * out_scale);
}

// scratch: 3 * tokens * W floats (only used by the chunked form)
XB_EXPORT int xb_gated_scan(int out_dtype, void* y, int ldy, const float* zxg, const float* bz, const float* bx, float* state,
                            const int* q_start, const int* slots, const int* req_of_token, int num_entries, int tokens,
                            int W, float out_scale, int chunked, float* scratch, cudaStream_t stream) {
    if (tokens <= 0 || num_entries <= 0) return 0;
    const int threads = 128;
    const unsigned cx = (unsigned)((W + threads - 1) / threads);
    typedef __nv_bfloat16 bf;
    if (!chunked || scratch == nullptr) {
        const dim3 grid(cx, num_entries);
        if (out_dtype == XB_F32)
            gated_scan_serial_kernel<float><<<grid, threads, 0, stream>>>((float*)y, ldy, zxg, bz, bx, state, q_start, slots, W, out_scale);
        else
            gated_scan_serial_kernel<bf><<<grid, threads, 0, stream>>>((bf*)y, ldy, zxg, bz, bx, state, q_start, slots, W, out_scale);
        return xb_launch_status();
    }
    float* prodA = scratch;
    float* endB = scratch + (size_t)tokens * W;
    float* start = scratch + 2 * (size_t)tokens * W;
    const int chunks = (tokens + GS_CH - 1) / GS_CH;
    gated_scan_chunk_kernel<<<dim3(cx, chunks), threads, 0, stream>>>(prodA, endB, zxg, bz, bx, req_of_token, tokens, W);
    int rc = xb_launch_status();
    if (rc) return rc;
    gated_scan_starts_kernel<<<dim3(cx, num_entries), threads, 0, stream>>>(start, prodA, endB, state, q_start, slots, W);
    rc = xb_launch_status();
    if (rc) return rc;
    if (out_dtype == XB_F32)
        gated_scan_finish_kernel<float><<<dim3(cx, tokens), threads, 0, stream>>>((float*)y, ldy, zxg, start, prodA, endB, req_of_token, q_start, tokens, W, out_scale);
    else
        gated_scan_finish_kernel<bf><<<dim3(cx, tokens), threads, 0, stream>>>((bf*)y, ldy, zxg, start, prodA, endB, req_of_token, q_start, tokens, W, out_scale);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Polynomial activation with normed powers, one block per row of F values:
//   act = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e,   rms(v) = sqrt(mean(v^2) + eps)
// coef = [a, b, c, e] on the device.
// ------------------------------------------------------------------------------------------
// Three sums over a block at once; every thread gets them.  Fixed order: lanes, then warps.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float* scratch /* 3 * 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; scratch[64 + warp] = c; }
    __syncthreads();
    a = warp_sum(lane < nwarps ? scratch[lane] : 0.f);
    b = warp_sum(lane < nwarps ? scratch[32 + lane] : 0.f);
    c = warp_sum(lane < nwarps ? scratch[64 + lane] : 0.f);
}

// PER values of the row per thread stay in registers between the sums and the result (F <= PER * threads).
template <typename T, int PER>
__global__ void polynorm_kernel(T* __restrict__ out, const float* __restrict__ z, const float* __restrict__ coef, int F,
                                float eps) {
    __shared__ float scratch[96];
    const float* zr = z + (size_t)blockIdx.x * F;
    float v[PER];
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < F ? zr[i] : 0.f;
        const float v2 = v[k] * v[k];
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    }
    block_sum3(s2, s4, s6, scratch);
    const float r1 = coef[0] / sqrtf(s2 / (float)F + eps);
    const float r2 = coef[1] / sqrtf(s4 / (float)F + eps);
    const float r3 = coef[2] / sqrtf(s6 / (float)F + eps);
    const float e = coef[3];
    T* o = out + (size_t)blockIdx.x * F;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const float v2 = v[k] * v[k];
        if (i < F) o[i] = from_f32<T>(v[k] * r1 + v2 * r2 + v2 * v[k] * r3 + e);
    }
}

// rows longer than 16 values per thread of the largest block: two passes over the row
template <typename T>
__global__ void polynorm_long_kernel(T* __restrict__ out, const float* __restrict__ z, const float* __restrict__ coef, int F,
                                     float eps) {
    __shared__ float scratch[96];
    const float* zr = z + (size_t)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    }
    block_sum3(s2, s4, s6, scratch);
    const float r1 = coef[0] / sqrtf(s2 / (float)F + eps);
    const float r2 = coef[1] / sqrtf(s4 / (float)F + eps);
    const float r3 = coef[2] / sqrtf(s6 / (float)F + eps);
    const float e = coef[3];
    T* o = out + (size_t)blockIdx.x * F;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        o[i] = from_f32<T>(v * r1 + v2 * r2 + v2 * v * r3 + e);
    }
}

template <typename T>
static int polynorm_launch(void* out, const float* z, const float* coef, int rows, int F, float eps, cudaStream_t stream) {
    if (F <= 4 * 256) polynorm_kernel<T, 4><<<rows, (F + 3) / 4 < 32 ? 32 : ((F + 3) / 4 + 31) / 32 * 32, 0, stream>>>((T*)out, z, coef, F, eps);
    else if (F <= 8 * 512) polynorm_kernel<T, 8><<<rows, ((F + 7) / 8 + 31) / 32 * 32, 0, stream>>>((T*)out, z, coef, F, eps);
    else if (F <= 16 * 1024) polynorm_kernel<T, 16><<<rows, ((F + 15) / 16 + 31) / 32 * 32, 0, stream>>>((T*)out, z, coef, F, eps);
    else polynorm_long_kernel<T><<<rows, 1024, 0, stream>>>((T*)out, z, coef, F, eps);
    return xb_launch_status();
}

XB_EXPORT int xb_polynorm(int out_dtype, void* out, const float* z, const float* coef, int rows, int F, float eps,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (out_dtype == XB_F32) return polynorm_launch<float>(out, z, coef, rows, F, eps, stream);
    return polynorm_launch<__nv_bfloat16>(out, z, coef, rows, F, eps, stream);
}
