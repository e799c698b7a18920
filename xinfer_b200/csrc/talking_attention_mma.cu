// The talking-heads attention (see talking_attention.cu for the arithmetic) for bfloat16 on tensor cores.
//
// The two products of a key tile - raw scores Q K^T and value sums P V - run as mma.sync m16n8k16 tiles;
// between them the scores of all heads meet on the FMA units: the mix across heads (heads^2 multiply-adds
// per query-key pair, float32, which no tensor-core mode computes in true 32-bit), the mask and the softmax
// rows.  That mix is why a block takes ALL heads of its queries, and it sets the kernel's floor: per pair
// 2 * heads * (d + dv) tensor-core operations stand beside 2 * heads^2 float32 operations on units that are
// some thirty times slower.
//
// A block takes `bq` consecutive queries of one entry.  The rows of kv head g are its group's query heads
// times the tile's queries (row = head_in_group * bq + query), padded to 16-row tiles; a (kv head, 16-row
// tile) pair is a unit, and the block's 8 warps share the units.  Per tile of 32 keys:
//   a. keys and values of every kv head to shared memory (16-byte asynchronous copies);
//   b. per unit: raw scores to shared memory [head][query][key];
//   c. one thread per (query, key): all heads' raw scores into registers, mixed by `talk`, masked;
//   d. one warp per (head, query) row: running maximum (0 at the start with a sink), weights, correction;
//   e. per unit: O <- O * correction + P V, O in registers.
#include "common.cuh"
#include "mma_sync.cuh"

using namespace xbmma;

__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

constexpr int TM_THREADS = 256;
constexpr int TM_WARPS = 8;
constexpr int TM_BK = 32;
constexpr int TM_LDS = TM_BK + 1;    // a score row's stride in shared memory: rows of one query tile fall into different banks

struct TalkMmaArgs {
    const int* q_start;
    const int* start_pos;
    const int* block_table;
    const float* talk;
    float* part_o;
    float* part_ml;
    int num_entries, table_stride, nh, nkv, d, dv, page_size, num_pages, window, sink, bq, parts, ldo, n_mt;
    float scale, out_scale;
    int* err;
};

struct TalkMmaSmem {
    // all offsets in bytes
    size_t q, k, v, s, p, talk, rm, rl, rc, total;
    int ldq, ldk, ldv, ldp, rows;   // element strides; rows = n_mt * 16
};

__host__ __device__ inline TalkMmaSmem talk_mma_smem(int H, int G, int d, int dv, int bq, int n_mt, int maxh) {
    TalkMmaSmem L;
    L.rows = n_mt * 16;
    L.ldq = d + 8; L.ldk = d + 8; L.ldv = dv + 8; L.ldp = TM_BK + 8;
    size_t at = 0;
    L.q = at; at += (size_t)G * L.rows * L.ldq * 2;
    L.k = at; at += (size_t)G * TM_BK * L.ldk * 2;
    L.v = at; at += (size_t)G * TM_BK * L.ldv * 2;
    L.p = at; at += (size_t)G * L.rows * L.ldp * 2;
    at = (at + 15) / 16 * 16;
    L.s = at; at += (size_t)H * bq * TM_LDS * 4;
    at = (at + 15) / 16 * 16;      // the mix matrix is read in 16-byte pieces
    L.talk = at; at += (size_t)maxh * maxh * 4;
    L.rm = at; at += (size_t)H * bq * 4;
    L.rl = at; at += (size_t)H * bq * 4;
    L.rc = at; at += (size_t)H * bq * 4;
    L.total = at;
    return L;
}

template <int MAXH, int DVT /* 8-column tiles of a value head */>
__global__ void __launch_bounds__(TM_THREADS) attn_talking_mma_kernel(__nv_bfloat16* __restrict__ out,
                                                                      const __nv_bfloat16* __restrict__ q,
                                                                      const __nv_bfloat16* __restrict__ k_cache,
                                                                      const __nv_bfloat16* __restrict__ v_cache,
                                                                      TalkMmaArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    __shared__ int s_entry, s_tile;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.nh, G = a.nkv, d = a.d, dv = a.dv, BQ = a.bq, rep = H / G, n_mt = a.n_mt;
    const int R = rep * BQ;                                  // real rows per kv head
    if (tid == 0) {
        int tile = blockIdx.x, found = -1;
        for (int b = 0; b < a.num_entries; ++b) {
            const int n = a.q_start[b + 1] - a.q_start[b];
            const int nt = (n + BQ - 1) / BQ;
            if (tile < nt) { found = b; break; }
            tile -= nt;
        }
        s_entry = found;
        s_tile = tile;
    }
    __syncthreads();
    const int b = s_entry;
    if (b < 0) return;
    const int n_b = a.q_start[b + 1] - a.q_start[b];
    const int i0 = s_tile * BQ;
    const int nq = min(BQ, n_b - i0);
    const int t0 = a.q_start[b] + i0;
    const int p0 = a.start_pos[b] + i0;
    const int* table = a.block_table + (size_t)b * a.table_stride;

    const TalkMmaSmem L = talk_mma_smem(H, G, d, dv, BQ, n_mt, MAXH);
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw + L.q);
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw + L.k);
    __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(smraw + L.v);
    __nv_bfloat16* Pb = reinterpret_cast<__nv_bfloat16*>(smraw + L.p);
    float* S = reinterpret_cast<float*>(smraw + L.s);        // [H][BQ][BK]
    float* tk = reinterpret_cast<float*>(smraw + L.talk);    // [MAXH][MAXH]
    float* rm = reinterpret_cast<float*>(smraw + L.rm);
    float* rl = reinterpret_cast<float*>(smraw + L.rl);
    float* rc = reinterpret_cast<float*>(smraw + L.rc);

    // queries: row r of kv head g is head g * rep + r / BQ, query r % BQ; rows beyond the real ones are zero
    const int dch = d / 8;                                   // 16-byte pieces of a head
    for (int e = tid; e < G * L.rows * dch; e += TM_THREADS) {
        const int c = e % dch, r = (e / dch) % L.rows, g = e / (dch * L.rows);
        const int hl = r / BQ, i = r - hl * BQ;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < R && i < nq)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + i) * H + (g * rep + hl)) * d + c * 8);
        *reinterpret_cast<uint4*>(Qs + ((size_t)g * L.rows + r) * L.ldq + c * 8) = v;
    }
    for (int e = tid; e < G * L.rows * (L.ldp / 8); e += TM_THREADS)
        reinterpret_cast<uint4*>(Pb)[e] = make_uint4(0, 0, 0, 0);      // padded rows stay zero
    for (int e = tid; e < MAXH * MAXH; e += TM_THREADS) {
        const int h = e / MAXH, g = e % MAXH;
        tk[e] = (h < H && g < H) ? (a.talk ? a.talk[h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    for (int e = tid; e < H * BQ; e += TM_THREADS) {
        rm[e] = a.sink && blockIdx.y == 0 ? 0.f : -INFINITY;
        rl[e] = a.sink && blockIdx.y == 0 ? 1.f : 0.f;
    }
    const int units = G * n_mt;
    constexpr int UMAX = 2;                                  // units a warp may own (host keeps units <= 2 * warps)
    float o[UMAX][DVT][4];
#pragma unroll
    for (int u = 0; u < UMAX; ++u)
#pragma unroll
        for (int n = 0; n < DVT; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) o[u][n][c] = 0.f;

    const int last = p0 + nq - 1;
    int lo = (a.window > 0 && p0 - a.window + 1 > 0) ? p0 - a.window + 1 : 0;
    int hi = last + 1;
    if (a.parts > 1) {
        const int base = lo / TM_BK * TM_BK;
        const int tiles = (hi - base + TM_BK - 1) / TM_BK;
        const int per = (tiles + a.parts - 1) / a.parts;
        const int first = base + (int)blockIdx.y * per * TM_BK;
        lo = max(lo, first);
        hi = min(hi, first + per * TM_BK);
    }
    const int vch = dv / 8;
    __shared__ int rowbase[2][TM_BK];          // per key of a tile: its row in the cache for kv head 0, or -1 ([0]: keys, [1]: values)
    const int bq_shift = 31 - __clz(BQ);       // BQ is a power of two

    // Rows of one tile are fetched by warps: a warp takes (kv head, key) rows in turn, its lanes the row's
    // 16-byte pieces.  Where the rows lie is worked out once per tile by 32 threads.
    auto find_rows = [&](int k0, int which) {
        if (tid < TM_BK) {
            const int key = k0 + tid;
            int rb = -1;
            if (key >= lo && key < hi) {
                const int page = table[key / a.page_size];
                if (page < 0 || page >= a.num_pages) atomicOr(a.err, XB_ERR_BAD_PAGE);
                else rb = page * G * a.page_size + key % a.page_size;
            }
            rowbase[which][tid] = rb;
        }
    };
    // a warp's lanes take the 16-byte pieces of one row, or of two rows at once where a row has at most 16 pieces
    auto fetch = [&](const __nv_bfloat16* cache, __nv_bfloat16* tile, const int* rows, int width, int ld, int pieces) {
        const int two = pieces <= 16 ? 1 : 0;
        const int sub = two ? lane >> 4 : 0, c0 = two ? lane & 15 : lane, step = two ? 16 : 32;
        const int per_pass = TM_WARPS << two;                 // rows the block's warps take at once
        // a thread meets the same few keys for every kv head: their rows are looked up once, the heads are strides
        for (int j = (warp << two) + sub; j < TM_BK; j += per_pass) {
            const int rb = rows[j];
            const bool ok = rb >= 0;
            const __nv_bfloat16* src = cache + (ok ? (size_t)rb * width : 0);
            const size_t src_step = ok ? (size_t)a.page_size * width : 0;
            uint32_t dst = smem_addr(tile + (size_t)j * ld);
            const uint32_t dst_step = (uint32_t)(TM_BK * ld * 2);
            for (int g = 0; g < G; ++g, src += src_step, dst += dst_step)
                for (int c = c0; c < pieces; c += step) cp_async16(dst + c * 16, src + c * 8, ok ? 16 : 0);
        }
        cp_async_commit();
    };
    auto fetch_keys = [&](void) { fetch(k_cache, Ks, rowbase[0], d, L.ldk, dch); };
    auto fetch_values = [&](void) { fetch(v_cache, Vs, rowbase[1], dv, L.ldv, vch); };
    const int k_first = lo / TM_BK * TM_BK;
    __syncthreads();                                        // the queries, the mix matrix and the rows' start values are in place
    if (k_first < hi) {
        find_rows(k_first, 0);
        find_rows(k_first, 1);
        __syncthreads();
        fetch_keys();
        fetch_values();
    }
    for (int k0 = k_first; k0 < hi; k0 += TM_BK) {
        // a. this tile's keys have been asked for (and its values behind them): wait for the keys
        cp_async_wait_but_one();
        __syncthreads();
        // b. raw scores per unit
        for (int u = warp; u < units; u += TM_WARPS) {
            const int g = u / n_mt, mt = u - g * n_mt;
            float acc[TM_BK / 8][4];
#pragma unroll
            for (int n = 0; n < TM_BK / 8; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[n][c] = 0.f;
            const __nv_bfloat16* qb = Qs + ((size_t)g * L.rows + mt * 16) * L.ldq;
            const __nv_bfloat16* kb = Ks + (size_t)g * TM_BK * L.ldk;
            for (int ks = 0; ks < d / 16; ++ks) {
                uint32_t af[4];
                ldmatrix_x4(af, smem_addr(qb + (size_t)(lane & 15) * L.ldq + ks * 16 + (lane >> 4) * 8));
#pragma unroll
                for (int nb = 0; nb < TM_BK / 16; ++nb) {
                    uint32_t bf[4];
                    ldmatrix_x4(bf, smem_addr(kb + (size_t)(nb * 16 + (lane & 7) + ((lane >> 4) << 3)) * L.ldk + ks * 16 + ((lane >> 3) & 1) * 8));
                    mma_bf16(acc[nb * 2], af, bf[0], bf[1]);
                    mma_bf16(acc[nb * 2 + 1], af, bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int n = 0; n < TM_BK / 8; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int r = mt * 16 + (lane >> 2) + (c >> 1) * 8;
                    const int j = n * 8 + (lane & 3) * 2 + (c & 1);
                    if (r < R) {
                        const int hl = r >> bq_shift, i = r & (BQ - 1);
                        S[((size_t)(g * rep + hl) * BQ + i) * TM_LDS + j] = acc[n][c] * a.scale;
                    }
                }
        }
        if (k0 + TM_BK < hi) find_rows(k0 + TM_BK, 0);
        __syncthreads();                                    // every warp is done with this tile's keys
        if (k0 + TM_BK < hi) fetch_keys();                  // the next tile's keys arrive during the mix, the softmax and P V
        else cp_async_commit();
        // c + d. a warp takes one query (all heads, or an interleaved share of them where the tile has fewer
        // queries than the block has warps), its lanes the tile's keys: every head's raw score of the pair into
        // registers, then head by head the mix, the mask, the row's running maximum, the weights and their sum
        {
            const int nsplit = BQ >= TM_WARPS ? 1 : TM_WARPS / BQ;
            for (int i = BQ >= TM_WARPS ? warp : (warp & (BQ - 1)); i < BQ; i += TM_WARPS) {
                const int key = k0 + lane, p = p0 + i;
                const bool seen = i < nq && key >= lo && key < hi && key <= p && (a.window <= 0 || key > p - a.window);
                float s[MAXH];
#pragma unroll
                for (int g = 0; g < MAXH; ++g) s[g] = g < H ? S[((size_t)g * BQ + i) * TM_LDS + lane] : 0.f;
#pragma unroll 1
                for (int h = BQ >= TM_WARPS ? 0 : (warp >> bq_shift); h < H; h += nsplit) {
                    const float4* tr = reinterpret_cast<const float4*>(tk + h * MAXH);
                    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
                    for (int g4 = 0; g4 < MAXH / 4; ++g4) {
                        const float4 t = tr[g4];
                        m0 = fmaf(t.x, s[g4 * 4], m0);
                        m1 = fmaf(t.y, s[g4 * 4 + 1], m1);
                        m2 = fmaf(t.z, s[g4 * 4 + 2], m2);
                        m3 = fmaf(t.w, s[g4 * 4 + 3], m3);
                    }
                    const float sv = seen ? (m0 + m1) + (m2 + m3) : -INFINITY;
                    const int r = h * BQ + i;
                    const float m_old = rm[r];
                    const float m_new = fmaxf(m_old, warp_max(sv));
                    const float w = m_new == -INFINITY ? 0.f : __expf(sv - m_new);
                    const __nv_bfloat16 wb = __float2bfloat16_rn(w);
                    const float sum = warp_sum(__bfloat162float(wb));    // the sum of the weights as the product sees them
                    const int g = h / rep, hl = h - g * rep;
                    Pb[((size_t)g * L.rows + hl * BQ + i) * L.ldp + lane] = wb;
                    __syncwarp();
                    if (lane == 0) {
                        rc[r] = m_new == -INFINITY ? 1.f : __expf(m_old - m_new);
                        rl[r] = rl[r] * rc[r] + sum;
                        rm[r] = m_new;
                    }
                }
            }
        }
        cp_async_wait_but_one();                            // this tile's values (the next keys may still be on their way)
        __syncthreads();
        // e. value sums per unit
#pragma unroll
        for (int uu = 0; uu < UMAX; ++uu) {
            const int u = warp + uu * TM_WARPS;
            if (u >= units) break;
            const int g = u / n_mt, mt = u - g * n_mt;
            float c0 = 1.f, c1 = 1.f;
            {
                const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
                if (r0 < R) c0 = rc[(g * rep + (r0 >> bq_shift)) * BQ + (r0 & (BQ - 1))];
                if (r1 < R) c1 = rc[(g * rep + (r1 >> bq_shift)) * BQ + (r1 & (BQ - 1))];
            }
#pragma unroll
            for (int n = 0; n < DVT; ++n) {
                o[uu][n][0] *= c0; o[uu][n][1] *= c0; o[uu][n][2] *= c1; o[uu][n][3] *= c1;
            }
            const __nv_bfloat16* pb = Pb + ((size_t)g * L.rows + mt * 16) * L.ldp;
            const __nv_bfloat16* vb = Vs + (size_t)g * TM_BK * L.ldv;
#pragma unroll
            for (int ks = 0; ks < TM_BK / 16; ++ks) {
                uint32_t af[4];
                ldmatrix_x4(af, smem_addr(pb + (size_t)(lane & 15) * L.ldp + ks * 16 + (lane >> 4) * 8));
#pragma unroll
                for (int nb = 0; nb < DVT / 2; ++nb) {
                    if (nb * 16 < dv) {
                        uint32_t bf[4];
                        ldmatrix_x4_trans(bf, smem_addr(vb + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * L.ldv + nb * 16 + (lane >> 4) * 8));
                        mma_bf16(o[uu][nb * 2], af, bf[0], bf[1]);
                        mma_bf16(o[uu][nb * 2 + 1], af, bf[2], bf[3]);
                    }
                }
            }
        }
        if (k0 + TM_BK < hi) find_rows(k0 + TM_BK, 1);
        __syncthreads();                                    // every warp is done with this tile's values, weights and scores
        if (k0 + TM_BK < hi) fetch_values();
        else cp_async_commit();
    }
    cp_async_wait_all();
    __syncthreads();
    // results: row r of unit (g, mt) is head g * rep + r / BQ of query r % BQ
#pragma unroll
    for (int uu = 0; uu < UMAX; ++uu) {
        const int u = warp + uu * TM_WARPS;
        if (u >= units) break;
        const int g = u / n_mt, mt = u - g * n_mt;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = mt * 16 + (lane >> 2) + half * 8;
            if (r >= R) continue;
            const int hl = r / BQ, i = r - hl * BQ, h = g * rep + hl;
            if (i >= nq) continue;
            if (a.parts > 1) {
                float* po = a.part_o + (((size_t)(t0 + i) * a.parts + blockIdx.y) * H + h) * dv;
#pragma unroll
                for (int n = 0; n < DVT; ++n) {
                    const int c = n * 8 + (lane & 3) * 2;
                    if (c < dv) {
                        po[c] = o[uu][n][half * 2];
                        po[c + 1] = o[uu][n][half * 2 + 1];
                    }
                }
                if ((lane & 3) == 0) {
                    float* pml = a.part_ml + (((size_t)(t0 + i) * a.parts + blockIdx.y) * H + h) * 2;
                    pml[0] = rm[h * BQ + i];
                    pml[1] = rl[h * BQ + i];
                }
            } else {
                const float l = rl[h * BQ + i];
                const float f = l > 0.f ? a.out_scale / l : 0.f;
                __nv_bfloat16* orow = out + (size_t)(t0 + i) * a.ldo + (size_t)h * dv;
#pragma unroll
                for (int n = 0; n < DVT; ++n) {
                    const int c = n * 8 + (lane & 3) * 2;
                    if (c < dv)
                        *reinterpret_cast<__nv_bfloat162*>(orow + c) = __floats2bfloat162_rn(o[uu][n][half * 2] * f, o[uu][n][half * 2 + 1] * f);
                }
            }
        }
    }
}

// defined in talking_attention.cu: puts a token's key ranges together
extern "C" int xb_attn_talking_merge_bf16(void* out, const float* part_o, const float* part_ml, int tokens, int H, int dv,
                                          int parts, int ldo, float out_scale, cudaStream_t stream);

// The query tile this kernel takes for these sizes (at most `want`), 0: the sizes are not for it (the FMA
// kernel takes them).  Needs head sizes in steps of 16 (values up to 128), at most 64 heads, an output row
// stride and head offsets that keep 4-byte stores aligned.
XB_EXPORT int xb_attn_talking_mma_tile(int nh, int nkv, int d, int dv, int want) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || nh > 64 || d % 16 || dv % 16 || d > 256 || dv > 128 || d < 16 || dv < 16) return 0;
    const int rep = nh / nkv;
    const int maxh = nh <= 8 ? 8 : (nh <= 16 ? 16 : (nh <= 32 ? 32 : 64));
    for (int bq = 16; bq >= 1; bq >>= 1) {
        if (bq > want && bq > 1) continue;
        const int n_mt = (rep * bq + 15) / 16;
        if (nkv * n_mt > 2 * TM_WARPS) continue;
        if (bq * TM_BK > 2 * TM_THREADS) continue;
        if (talk_mma_smem(nh, nkv, d, dv, bq, n_mt, maxh).total > 220 * 1024) continue;
        return bq;
    }
    return 0;
}

template <int MAXH, int DVT>
static int talk_mma_launch(void* out, const void* q, const void* kc, const void* vc, const TalkMmaArgs& a, dim3 grid, size_t smem,
                           cudaStream_t stream) {
    typedef __nv_bfloat16 bf;
    cudaFuncSetAttribute(attn_talking_mma_kernel<MAXH, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attn_talking_mma_kernel<MAXH, DVT><<<grid, TM_THREADS, smem, stream>>>((bf*)out, (const bf*)q, (const bf*)kc, (const bf*)vc, a);
    return xb_launch_status();
}

XB_EXPORT int xb_attn_talking_mma(void* out, int ldo, const void* q, const void* k_cache, const void* v_cache, const float* talk,
                                  const int* q_start, const int* start_pos, int num_entries, const int* block_table,
                                  int table_stride, int tokens, int nh, int nkv, int d, int dv, int page_size, int num_pages,
                                  int window, float scale, int sink, float out_scale, int bq, int parts, float* part_o,
                                  float* part_ml, int* err, cudaStream_t stream) {
    if (tokens <= 0 || num_entries <= 0) return 0;
    if (bq <= 0 || xb_attn_talking_mma_tile(nh, nkv, d, dv, bq) < bq || (ldo % 2) || (((uintptr_t)out) & 3))
        return (int)cudaErrorInvalidValue;
    if (parts > 1 && (!part_o || !part_ml)) return (int)cudaErrorInvalidValue;
    const int rep = nh / nkv;
    TalkMmaArgs a;
    a.q_start = q_start; a.start_pos = start_pos; a.block_table = block_table; a.talk = talk;
    a.part_o = part_o; a.part_ml = part_ml;
    a.num_entries = num_entries; a.table_stride = table_stride; a.nh = nh; a.nkv = nkv; a.d = d; a.dv = dv;
    a.page_size = page_size; a.num_pages = num_pages; a.window = window; a.sink = sink; a.bq = bq;
    a.parts = parts < 1 ? 1 : parts; a.ldo = ldo; a.n_mt = (rep * bq + 15) / 16;
    a.scale = scale; a.out_scale = out_scale; a.err = err;
    const int maxh = nh <= 8 ? 8 : (nh <= 16 ? 16 : (nh <= 32 ? 32 : 64));
    const size_t smem = talk_mma_smem(nh, nkv, d, dv, bq, a.n_mt, maxh).total;
    const dim3 grid((tokens + bq - 1) / bq + num_entries, a.parts);
    const bool wide = dv > 64;
    int rc;
#define XB_TM(MH)                                                                                                   \
    rc = wide ? talk_mma_launch<MH, 16>(out, q, k_cache, v_cache, a, grid, smem, stream)                            \
              : talk_mma_launch<MH, 8>(out, q, k_cache, v_cache, a, grid, smem, stream)
    if (maxh == 8) XB_TM(8);
    else if (maxh == 16) XB_TM(16);
    else if (maxh == 32) XB_TM(32);
    else XB_TM(64);
#undef XB_TM
    if (rc == 0 && a.parts > 1)
        rc = xb_attn_talking_merge_bf16(out, part_o, part_ml, tokens, nh, dv, a.parts, ldo, out_scale, stream);
    return rc;
}
