// Attention over cached latent rows on tensor cores (bfloat16, mma.sync m16n8k16, float32 accumulators).
//
// Every head of every token attends over the SAME cached rows [c | k_r] (dk = rank + rot channels; the first
// `rank` channels are also the value), so the (token, head) pairs of a request are simply rows of one tall
// query matrix: row = token * heads + head, exactly how the queries lie in memory.  A block takes 16 * RG
// consecutive rows of one entry and walks over the keys they see in tiles of 64:
//
//   a. the tile's cached rows to shared memory by 16-byte asynchronous copies, one tile ahead (two buffers);
//      rows outside the request are zero-filled;
//   b. S = Q K^T: the warps of a row group take 16 (or 8) keys each; a warp runs over the dk channels in four
//      interleaved streams with accumulators of their own (eight independent accumulator tiles, so that no
//      product waits for the one before it) and adds them at the end; the scores go to shared memory as float32;
//   c. every warp reads its row group's scores in the layout of an A operand, scales them (into the base-2
//      domain: weights are exp2), masks them where the tile touches a causal or window edge (tiles that every
//      row of the block sees whole skip the masks), and keeps the running maximum and sum of its rows (the four
//      warps of a row group compute the same numbers); a head's sink enters as the start of maximum and sum;
//   d. O <- O * correction + P V: the warps of a row group take the value columns in turn (8-column tiles
//      c, c + CW, c + 2 CW, ...), so a row's accumulators are spread over the warps and a latent of 512
//      channels fits in registers.
// A row group has four warps, or eight for wide latents (the block then has up to 16 warps over the same tiles
// in shared memory: the tiles allow one block per SM, and more warps hide each other's waits).
//
// With `parts` > 1 (single tokens over long contexts) a row's key tiles are dealt out to `parts` blocks, which
// leave unnormed sums, maxima and denominators in scratch; attn_latent_merge_kernel joins them.
#include "common.cuh"
#include "mma_sync.cuh"

using namespace xbmma;

namespace {

__device__ __forceinline__ void cp_async_wait_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

constexpr int LM_BK = 64;            // keys per tile
constexpr int LM_LDS = LM_BK + 8;    // floats per score row in shared memory

struct LatentMmaArgs {
    const int* q_start;
    const int* start_pos;
    const int* block_table;
    const float* sink;
    float* part_o;
    float* part_ml;
    int num_entries, table_stride, nh, dk, rank, page_size, num_pages, window, parts, rg;
    float scale;
    int* err;
};

__host__ __device__ inline size_t latent_mma_smem(int dk, int rg) {
    const size_t ld = dk + 8;
    return (size_t)(16 * rg + 2 * LM_BK) * ld * 2 + (size_t)16 * rg * LM_LDS * 4;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}

template <int MAXNT /* 8-column value tiles per warp */, int CW /* warps of a row group: 4 or 8 */>
__global__ void __launch_bounds__(64 * CW) attn_latent_mma_kernel(__nv_bfloat16* __restrict__ out,
                                                              const __nv_bfloat16* __restrict__ q,
                                                              const __nv_bfloat16* __restrict__ cache, LatentMmaArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    __shared__ int s_entry, s_tile;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.nh, dk = a.dk, rank = a.rank, R = 16 * a.rg;
    const int rgi = warp / CW, cw = warp % CW;               // row group and column warp
    constexpr int KW = LM_BK / CW;                          // keys of a warp in Q K^T: 16 or 8
    if (tid == 0) {
        int tile = blockIdx.x, found = -1;
        for (int b = 0; b < a.num_entries; ++b) {
            const int rows = (a.q_start[b + 1] - a.q_start[b]) * H;
            const int nt = (rows + R - 1) / R;
            if (tile < nt) { found = b; break; }
            tile -= nt;
        }
        s_entry = found;
        s_tile = tile;
    }
    __syncthreads();
    const int b = s_entry;
    if (b < 0) return;
    const int count = a.q_start[b + 1] - a.q_start[b];
    const int row0 = s_tile * R;                            // first row of the block within the entry
    const int nrows = min(R, count * H - row0);
    const int start = a.start_pos[b];
    const size_t grow0 = (size_t)a.q_start[b] * H + row0;   // first row among all rows of the step
    const int p_lo = start + row0 / H, p_hi = start + (row0 + nrows - 1) / H;
    const int k_begin = (a.window > 0 && p_lo - a.window + 1 > 0) ? p_lo - a.window + 1 : 0;
    const int n_tiles = (p_hi - k_begin) / LM_BK + 1;
    const int part = blockIdx.y;
    const int per = (n_tiles + a.parts - 1) / a.parts;
    const int t_lo = part * per, t_hi = min(n_tiles, t_lo + per);
    const int* table = a.block_table + (size_t)b * a.table_stride;

    const int ld = dk + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);
    __nv_bfloat16* Ks = Qs + (size_t)R * ld;                // two buffers of LM_BK rows
    float* Ss = reinterpret_cast<float*>(Ks + (size_t)2 * LM_BK * ld);

    const int chunks = dk / 8;                              // 16-byte pieces of a row
    for (int e = tid; e < R * chunks; e += blockDim.x) {
        const int r = e / chunks, c = e - r * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (grow0 + r) * dk + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)r * ld + c * 8) = v;
    }

    const int nwarps = blockDim.x >> 5;
    // a warp per cached row (one page lookup), its lanes over the row's 16-byte pieces
    auto fetch = [&](int t, int buf) {
        const int k0 = k_begin + t * LM_BK;
        __nv_bfloat16* dst = Ks + (size_t)buf * LM_BK * ld;
        // the pages of this warp's rows (r = warp, warp + nwarps, ...), one lane each: the lookups wait together
        int my_page = -2;
        {
            const int j = k0 + warp + lane * nwarps;
            if (warp + lane * nwarps < LM_BK && j <= p_hi) my_page = table[j / a.page_size];
        }
        for (int r = warp, i = 0; r < LM_BK; r += nwarps, ++i) {
            const int j = k0 + r;
            const int page = __shfl_sync(0xffffffffu, my_page, i);
            const __nv_bfloat16* src = nullptr;
            if (j <= p_hi) {
                if (page < 0 || page >= a.num_pages) {
                    if (lane == 0) atomicOr(a.err, XB_ERR_BAD_PAGE);
                } else {
                    src = cache + ((size_t)page * a.page_size + (j % a.page_size)) * dk;
                }
            }
            const uint32_t d0 = smem_addr(dst + (size_t)r * ld);
            for (int c = lane; c < chunks; c += 32)
                cp_async16(d0 + c * 16, src ? src + c * 8 : cache, src ? 16 : 0);
        }
        cp_async_commit();
    };

    // this thread's two rows (lane / 4 and lane / 4 + 8 of the row group): position, head, running maximum and sum
    const int quad = lane & 3;
    int rpos[2];
    float m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rgi * 16 + (lane >> 2) + 8 * i;
        const bool valid = r < nrows;
        rpos[i] = valid ? start + (row0 + r) / H : -1;      // a row beyond the entry sees no key
        m[i] = -INFINITY;
        l[i] = 0.f;
        if (valid && a.sink != nullptr && part == 0) {      // the entry without a key: exp(sink - m) with m = sink
            m[i] = a.sink[(row0 + r) % H] * 1.4426950408889634f;    // maxima are kept in the base-2 domain
            l[i] = 1.f;
        }
    }
    float o[MAXNT][4];
#pragma unroll
    for (int n = 0; n < MAXNT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int ntiles_v = rank / 8;

    if (t_lo < t_hi) fetch(t_lo, 0);
    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) {
            fetch(t + 1, buf ^ 1);
            cp_async_wait_one();
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        const __nv_bfloat16* Kt = Ks + (size_t)buf * LM_BK * ld;
        const int k0 = k_begin + t * LM_BK;

        // b. scores of this warp's keys (16, or 8 with eight warps to a row group): four streams over the channels,
        //    each with accumulators of its own
        {
            constexpr int NT = KW / 8;     // 8-key tiles of this warp
            float s[4][NT][4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int n = 0; n < NT; ++n) s[u][n][0] = s[u][n][1] = s[u][n][2] = s[u][n][3] = 0.f;
            const int mi = lane >> 3, rr = lane & 7;
            const uint32_t qa = smem_addr(Qs + (size_t)(rgi * 16 + (mi & 1) * 8 + rr) * ld + (mi >> 1) * 8);
            const int steps = dk / 16;
            int ks = 0;
            if (NT == 2) {
                // one load brings 16 keys x 16 channels: the B operands of two key tiles for one step
                const uint32_t ka = smem_addr(Kt + (size_t)(cw * KW + (mi >> 1) * 8 + rr) * ld + (mi & 1) * 8);
                for (; ks + 4 <= steps; ks += 4) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t af[4], bf[4];
                        ldmatrix_x4(af, qa + (ks + u) * 32);
                        ldmatrix_x4(bf, ka + (ks + u) * 32);
                        mma_bf16(s[u][0], af, bf[0], bf[1]);
                        mma_bf16(s[u][NT - 1], af, bf[2], bf[3]);
                    }
                }
                for (; ks < steps; ++ks) {
                    uint32_t af[4], bf[4];
                    ldmatrix_x4(af, qa + ks * 32);
                    ldmatrix_x4(bf, ka + ks * 32);
                    mma_bf16(s[0][0], af, bf[0], bf[1]);
                    mma_bf16(s[0][NT - 1], af, bf[2], bf[3]);
                }
            } else {
                // one load brings 8 keys x 32 channels: the B operands of one key tile for two steps
                const uint32_t ka = smem_addr(Kt + (size_t)(cw * KW + rr) * ld + mi * 8);
                for (; ks + 4 <= steps; ks += 4) {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        uint32_t a0[4], a1[4], bf[4];
                        ldmatrix_x4(a0, qa + (ks + 2 * u) * 32);
                        ldmatrix_x4(a1, qa + (ks + 2 * u + 1) * 32);
                        ldmatrix_x4(bf, ka + (ks + 2 * u) * 32);
                        mma_bf16(s[2 * u][0], a0, bf[0], bf[1]);
                        mma_bf16(s[2 * u + 1][0], a1, bf[2], bf[3]);
                    }
                }
                for (; ks + 2 <= steps; ks += 2) {
                    uint32_t a0[4], a1[4], bf[4];
                    ldmatrix_x4(a0, qa + ks * 32);
                    ldmatrix_x4(a1, qa + (ks + 1) * 32);
                    ldmatrix_x4(bf, ka + ks * 32);
                    mma_bf16(s[0][0], a0, bf[0], bf[1]);
                    mma_bf16(s[1][0], a1, bf[2], bf[3]);
                }
                if (ks < steps) {          // an odd last step: the load's second half lies in the row's padding and is not used
                    uint32_t a0[4], bf[4];
                    ldmatrix_x4(a0, qa + ks * 32);
                    ldmatrix_x4(bf, ka + ks * 32);
                    mma_bf16(s[0][0], a0, bf[0], bf[1]);
                }
            }
            float* srow = Ss + (size_t)(rgi * 16 + (lane >> 2)) * LM_LDS + cw * KW + 2 * quad;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                float c[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) c[e] = (s[0][n][e] + s[1][n][e]) + (s[2][n][e] + s[3][n][e]);
                *reinterpret_cast<float2*>(srow + n * 8) = make_float2(c[0], c[1]);
                *reinterpret_cast<float2*>(srow + 8 * LM_LDS + n * 8) = make_float2(c[2], c[3]);
            }
        }
        __syncthreads();

        // c. running maximum and weights of this thread's two rows in the layout of an A operand (base-2 domain)
        // every row of the block sees every key of the tile: no masks
        const bool whole = k0 + LM_BK - 1 <= p_lo && (a.window <= 0 || k0 > p_hi - a.window) && nrows == R;
        const float sc2 = a.scale * 1.4426950408889634f;
        float p[2][16];
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float* srow = Ss + (size_t)(rgi * 16 + (lane >> 2) + 8 * i) * LM_LDS;
            float mx = -INFINITY;
            if (whole) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const float2 v = *reinterpret_cast<const float2*>(srow + kk * 16 + hf * 8 + 2 * quad);
                        const float x0 = v.x * sc2, x1 = v.y * sc2;
                        p[i][kk * 4 + hf * 2] = x0;
                        p[i][kk * 4 + hf * 2 + 1] = x1;
                        mx = fmaxf(mx, fmaxf(x0, x1));
                    }
            } else {
                // keys this row sees within the tile: columns lo .. hi
                const int hi = rpos[i] - k0;
                const int lo = a.window > 0 ? rpos[i] - a.window + 1 - k0 : -0x40000000;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const int col = kk * 16 + hf * 8 + 2 * quad;
                        const float2 v = *reinterpret_cast<const float2*>(srow + col);
                        const float x0 = (col >= lo && col <= hi) ? v.x * sc2 : -INFINITY;
                        const float x1 = (col + 1 >= lo && col + 1 <= hi) ? v.y * sc2 : -INFINITY;
                        p[i][kk * 4 + hf * 2] = x0;
                        p[i][kk * 4 + hf * 2 + 1] = x1;
                        mx = fmaxf(mx, fmaxf(x0, x1));
                    }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[i], mx);
            const float base = m_new == -INFINITY ? 0.f : m_new;     // nothing seen yet: every weight is zero
            corr[i] = exp2f(m[i] - base);
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                p[i][e] = exp2f(p[i][e] - base);
                sum += p[i][e];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[i] = l[i] * corr[i] + sum;
            m[i] = m_new;
        }

        // d. value sums of this warp's column tiles
#pragma unroll
        for (int n = 0; n < MAXNT; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
#pragma unroll
        for (int kp = 0; kp < 2; ++kp) {          // two 16-key steps per load
            uint32_t pa[2][4];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const int kk = kp * 2 + h2;
                pa[h2][0] = pack_bf16(p[0][kk * 4 + 0], p[0][kk * 4 + 1]);
                pa[h2][1] = pack_bf16(p[1][kk * 4 + 0], p[1][kk * 4 + 1]);
                pa[h2][2] = pack_bf16(p[0][kk * 4 + 2], p[0][kk * 4 + 3]);
                pa[h2][3] = pack_bf16(p[1][kk * 4 + 2], p[1][kk * 4 + 3]);
            }
            const uint32_t va = smem_addr(Kt + (size_t)(kp * 32 + lane) * ld);
#pragma unroll
            for (int n = 0; n < MAXNT; ++n) {
                const int nt = cw + CW * n;
                if (nt < ntiles_v) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, va + nt * 16);
                    mma_bf16(o[n], pa[0], vf[0], vf[1]);
                    mma_bf16(o[n], pa[1], vf[2], vf[3]);
                }
            }
        }
        __syncthreads();
    }

    // epilogue
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rgi * 16 + (lane >> 2) + 8 * i;
        if (r >= nrows) continue;
        const size_t grow = grow0 + r;
        if (a.parts > 1) {
            float* po = a.part_o + (grow * a.parts + part) * rank;
#pragma unroll
            for (int n = 0; n < MAXNT; ++n) {
                const int nt = cw + CW * n;
                if (nt < ntiles_v) *reinterpret_cast<float2*>(po + nt * 8 + 2 * quad) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
            }
            if (cw == 0 && quad == 0) {
                a.part_ml[(grow * a.parts + part) * 2] = m[i];
                a.part_ml[(grow * a.parts + part) * 2 + 1] = l[i];
            }
        } else {
            const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
            __nv_bfloat16* orow = out + grow * rank;
#pragma unroll
            for (int n = 0; n < MAXNT; ++n) {
                const int nt = cw + CW * n;
                if (nt < ntiles_v)
                    *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8 + 2 * quad) =
                        __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            }
        }
    }
}

// out[row] = sum_p part_o[row, p] 2^(m_p - M) / sum_p l_p 2^(m_p - M),  M = max_p m_p  (maxima in the base-2 domain)
__global__ void attn_latent_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, int parts, int rank) {
    const size_t row = blockIdx.x;
    float M = -INFINITY;
    for (int p = 0; p < parts; ++p) M = fmaxf(M, part_ml[(row * parts + p) * 2]);
    float L = 0.f;
    for (int p = 0; p < parts; ++p) {
        const float mp = part_ml[(row * parts + p) * 2];
        if (mp > -INFINITY) L += part_ml[(row * parts + p) * 2 + 1] * exp2f(mp - M);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
        for (int p = 0; p < parts; ++p) {
            const float mp = part_ml[(row * parts + p) * 2];
            if (mp > -INFINITY) acc += part_o[(row * parts + p) * rank + c] * exp2f(mp - M);
        }
        out[row * rank + c] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

// 1 when the tensor-core form takes these sizes (bfloat16 only), else 0.
XB_EXPORT int xb_attn_latent_mma_takes(int dk, int rank) {
    return dk % 16 == 0 && rank % 8 == 0 && rank > 0 && rank <= dk && rank <= 512 && latent_mma_smem(dk, 2) <= 227 * 1024;
}

// q [tokens, heads, dk], cache [pages, page_size, dk], out [tokens, heads, rank], all bfloat16.  `rg`: 16-row
// groups per block (1 or 2).  `parts` > 1 needs part_o (tokens * heads * parts * rank floats) and part_ml
// (tokens * heads * parts * 2 floats).
XB_EXPORT int xb_attn_latent_mma(void* out, const void* q, const void* cache, const int* q_start, const int* start_pos,
                                 int num_entries, const int* block_table, int table_stride, int tokens, int nh, int dk,
                                 int rank, int page_size, int num_pages, int window, float scale, const float* sink, int rg,
                                 int parts, float* part_o, float* part_ml, int* err, cudaStream_t stream) {
    if (tokens <= 0 || num_entries <= 0) return 0;
    if (!xb_attn_latent_mma_takes(dk, rank) || (rg != 1 && rg != 2) || parts < 1 || parts > 65535) return (int)cudaErrorInvalidValue;
    if (parts > 1 && (part_o == nullptr || part_ml == nullptr)) return (int)cudaErrorInvalidValue;
    LatentMmaArgs a;
    a.q_start = q_start; a.start_pos = start_pos; a.block_table = block_table; a.sink = sink;
    a.part_o = part_o; a.part_ml = part_ml;
    a.num_entries = num_entries; a.table_stride = table_stride; a.nh = nh; a.dk = dk; a.rank = rank;
    a.page_size = page_size; a.num_pages = num_pages; a.window = window; a.parts = parts; a.rg = rg;
    a.scale = scale; a.err = err;
    const int R = 16 * rg;
    // every entry's rows are cut into tiles of their own: at most one ragged tile per entry
    const long long tiles = ((long long)tokens * nh + R - 1) / R + num_entries;
    const size_t smem = latent_mma_smem(dk, rg);
    // eight warps to a row group where the latent is wide (more warps to hide each other's waits over the same tiles
    // in shared memory), four where a warp would be left with less than two value tiles
    const int cw = rank >= 128 ? 8 : 4;
    const dim3 grid((unsigned)tiles, (unsigned)parts), block(32 * cw * rg);
    const int ntw = (rank / 8 + cw - 1) / cw;      // value tiles per warp
#define XB_GO(N, C)                                                                                                  \
    do {                                                                                                             \
        cudaFuncSetAttribute(attn_latent_mma_kernel<N, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        attn_latent_mma_kernel<N, C><<<grid, block, smem, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)q,    \
                                                                    (const __nv_bfloat16*)cache, a);                 \
    } while (0)
    if (cw == 8) {
        if (ntw <= 2) XB_GO(2, 8);
        else if (ntw <= 4) XB_GO(4, 8);
        else XB_GO(8, 8);
    } else {
        if (ntw <= 2) XB_GO(2, 4);
        else XB_GO(4, 4);
    }
#undef XB_GO
    int rc = xb_launch_status();
    if (rc != 0 || parts == 1) return rc;
    attn_latent_merge_kernel<<<(unsigned)((long long)tokens * nh), 128, 0, stream>>>((__nv_bfloat16*)out, part_o, part_ml, parts, rank);
    return xb_launch_status();
}
