// Attention in the latent space on the tensor cores (bf16, warp-level MMA), for prompt portions and
// single decoded tokens alike.
//
// All H query heads of a token read the same cache rows [rank + rot]; the value of a row is its
// leading rank columns.  So the H heads of consecutive tokens are the rows of one query tile: row
// i of an entry is (token i / H, head i % H), its position is that token's, and every key tile in
// shared memory serves all of them, once as K (scores, over all columns) and once as V (weighted
// sum, over the leading columns, read transposed).  A decoded token is a tile of H rows; a portion
// of n tokens has n * H rows in tiles of 64.
//
// One kernel, two shapes, each launch skipping the other's entries.  Entries of more than 16 rows:
// tiles of 64 rows, 16 per warp, every warp over all keys of a key tile; a request's last tile comes
// first, since it has the most keys.  Entries of one token (a decoded token: its heads in tiles of 16)
// or of at most 16 rows: tiles of 16 rows that all four warps share, each warp taking 16 of a key
// tile's 64 keys with running sums of its own, merged through shared memory at the end.  The keys of a tile may be cut
// into `splits` slices (grid.y); every slice leaves (max, sum, weighted sum) in scratch and a second
// kernel merges them.  Key tiles of 64 rows come in by cp.async through the block table (a warp per
// row, one page look-up per row), two buffers.  Scores, softmax statistics and sums are float.
//
// Widths are run-time numbers below compile-time bounds (two instantiations: up to 128 + 128 and
// up to 256 key / 192 value columns); rank + rot a multiple of 16, rank a multiple of 8.
#include "common.cuh"

namespace {

// keys per tile, for both tile shapes (32-key tiles for the 64-row shape, which let three CTAs share an
// SM instead of two, measured slower: 309 against 294 us for a prompt of 2,048 tokens)
template <bool SMALL> struct KeyTile { static constexpr int value = 64; };

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;                    // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The tile'th query tile among the entries that this launch takes (small: entries of one token or
// of at most 16 rows; else the others): its entry and first row.  False beyond the last one.
__device__ __forceinline__ bool find_tile(int tile, const int* __restrict__ cu_q, int n_entries, int heads,
                                          int rows_per_tile, bool small, int& entry, int& row0) {
    for (int e = 0; e < n_entries; ++e) {
        const int q_len = cu_q[e + 1] - cu_q[e], rows = q_len * heads;
        if (rows <= 0 || (q_len == 1 || rows <= 16) != small) continue;
        const int tiles = (rows + rows_per_tile - 1) / rows_per_tile;
        if (tile < tiles) {
            entry = e;
            row0 = (small ? tile : tiles - 1 - tile) * rows_per_tile;     // the tile with the most keys first
            return true;
        }
        tile -= tiles;
    }
    return false;
}

template <bool SMALL, int MAXDK16, int MAXDV8>
__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                       float* __restrict__ part_o, float* __restrict__ part_ml,
                       const __nv_bfloat16* __restrict__ pool, const int* __restrict__ cu_q,
                       const int* __restrict__ kv_len, const int* __restrict__ block_table, int max_blocks,
                       int num_pages, int page_shift, int n_entries, int heads, int dk, int dv, float scale,
                       int* err) {
    constexpr int WARPS = 4;
    constexpr int KT = KeyTile<SMALL>::value;
    constexpr int BM = SMALL ? 16 : 64;               // query rows of a tile
    constexpr int NT = SMALL ? 2 : KT / 8;            // blocks of 8 keys that a warp takes of a key tile
    const int page_size = 1 << page_shift;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ld = dk + 8;                            // padded row: ldmatrix without bank conflicts
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [BM][ld]
    __nv_bfloat16* k_s = q_s + BM * ld;                                          // [2][KT][ld]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int dk16 = dk >> 4, dv8 = dv >> 3;
    pdl_launch_dependents();
    int entry, row0;
    if (!find_tile(blockIdx.x, cu_q, n_entries, heads, BM, SMALL, entry, row0)) return;
    const int splits = gridDim.y, split = blockIdx.y;
    const int wrow = SMALL ? 0 : warp * 16;           // the warp's first row of the tile
    const int wkey = SMALL ? warp * 16 : 0;           // and its first key of a key tile
    const int q_first = cu_q[entry], q_len = cu_q[entry + 1] - q_first, kv = kv_len[entry];
    const int rows = q_len * heads;
    const int n_rows = min(BM, rows - row0);
    const int pos0 = kv - q_len;                      // position of the entry's first token
    const int last_tok = (row0 + n_rows - 1) / heads;
    const int n_keys = pos0 + last_tok + 1;           // keys that the tile's last row sees
    const int key_tiles = (n_keys + KT - 1) / KT;
    const int per = (key_tiles + splits - 1) / splits;
    const int kt_lo = split * per, kt_hi = min(key_tiles, kt_lo + per);
    const int* table = block_table + (long long)entry * max_blocks;
    const int chunks = dk >> 3;                       // 16-byte pieces of a row
    pdl_wait();

    // the tile's query rows (rows beyond the entry's: zeros)
    for (int r = warp; r < BM; r += WARPS) {
        const bool ok = r < n_rows;
        const long long src = ok ? ((long long)q_first * heads + row0 + r) * dk : 0;
        for (int c = lane; c < chunks; c += 32) cp_async16(q_s + r * ld + c * 8, q + src + c * 8, ok);
    }
    bool bad_page = false;
    auto load_keys = [&](int kt, int buf) {
        __nv_bfloat16* dst = k_s + buf * KT * ld;
        for (int r = warp; r < KT; r += WARPS) {
            const int j = kt * KT + r;
            bool ok = j < n_keys;
            long long src = 0;
            if (ok) {
                const int page = table[j >> page_shift];
                if (page < 0 || page >= num_pages) {
                    bad_page = true;
                    ok = false;
                } else {
                    src = (((long long)page << page_shift) + (j & (page_size - 1))) * dk;
                }
            }
            for (int c = lane; c < chunks; c += 32) cp_async16(dst + r * ld + c * 8, pool + src + c * 8, ok);
        }
    };
    if (kt_lo < kt_hi) load_keys(kt_lo, 0);
    cp_async_commit();

    float o_acc[MAXDV8][4];
#pragma unroll
    for (int i = 0; i < MAXDV8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // this thread's two rows (g and g + 8 of the warp's 16) and the last key each may see
    const int r_a = wrow + g, r_b = r_a + 8;
    const int see_a = pos0 + (row0 + min(r_a, n_rows - 1)) / heads;
    const int see_b = pos0 + (row0 + min(r_b, n_rows - 1)) / heads;
    const float sl2 = scale * 1.4426950408889634f;   // scores in units of log2 e

    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt + 1 < kt_hi) load_keys(kt + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kb = k_s + buf * KT * ld;
        // S = Q K^T for the warp's 16 rows and its keys of the tile
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < MAXDK16; ++ks) {
            if (ks < dk16) {
                uint32_t a0, a1, a2, a3;
                ldsm_x4(a0, a1, a2, a3, q_s + (wrow + (lane & 15)) * ld + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int j = 0; j < NT / 2; ++j) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(b0, b1, b2, b3, kb + (wkey + j * 16 + (lane & 7) + (lane >> 4) * 8) * ld + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * j], a0, a1, a2, a3, b0, b1);
                    mma_bf16(s[2 * j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        // causal mask, running maximum and sum
        const int key0 = kt * KT + wkey + 2 * t4;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int k0 = key0 + j * 8;
            s[j][0] = k0 <= see_a ? s[j][0] * sl2 : -INFINITY;
            s[j][1] = k0 + 1 <= see_a ? s[j][1] * sl2 : -INFINITY;
            s[j][2] = k0 <= see_b ? s[j][2] * sl2 : -INFINITY;
            s[j][3] = k0 + 1 <= see_b ? s[j][3] * sl2 : -INFINITY;
            mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float new_a = fmaxf(m_run[0], mx_a), new_b = fmaxf(m_run[1], mx_b);
        const float base_a = new_a == -INFINITY ? 0.f : new_a, base_b = new_b == -INFINITY ? 0.f : new_b;
        const float corr_a = exp2f(m_run[0] - base_a), corr_b = exp2f(m_run[1] - base_b);   // 0 while nothing was seen
        m_run[0] = new_a;
        m_run[1] = new_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            s[j][0] = exp2f(s[j][0] - base_a);
            s[j][1] = exp2f(s[j][1] - base_a);
            s[j][2] = exp2f(s[j][2] - base_b);
            s[j][3] = exp2f(s[j][3] - base_b);
            sum_a += s[j][0] + s[j][1];
            sum_b += s[j][2] + s[j][3];
        }
        l_run[0] = l_run[0] * corr_a + sum_a;          // (the quad's partial sums are added at the end)
        l_run[1] = l_run[1] * corr_b + sum_b;
#pragma unroll
        for (int i = 0; i < MAXDV8; ++i) {
            o_acc[i][0] *= corr_a;
            o_acc[i][1] *= corr_a;
            o_acc[i][2] *= corr_b;
            o_acc[i][3] *= corr_b;
        }
        // O += P V, V the leading dv columns of the same rows, read transposed
#pragma unroll
        for (int kk = 0; kk < NT / 2; ++kk) {
            const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < (MAXDV8 + 1) / 2; ++n2) {
                if (2 * n2 < dv8) {
                    uint32_t b0, b1, b2, b3;
                    // (a second block of 8 columns beyond dv is still inside the row: dk >= dv + ... or the row's padding)
                    ldsm_x4_t(b0, b1, b2, b3, kb + (wkey + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n2 * 16 + (lane >> 4) * 8);
                    mma_bf16(o_acc[2 * n2], a0, a1, a2, a3, b0, b1);
                    if (2 * n2 + 1 < MAXDV8 && 2 * n2 + 1 < dv8) mma_bf16(o_acc[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();                               // the buffer is free for the tile after next
    }
    cp_async_wait<0>();
    if (__syncthreads_or(bad_page ? 1 : 0) && threadIdx.x == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);

    if (SMALL) {
        // the four warps hold sums over different keys of the same 16 rows: warps 1..3 leave theirs in
        // shared memory (the key buffers are free now), warp 0 adds them to its own in warp order
        float* xo = reinterpret_cast<float*>(k_s);                  // [3][16][dv]
        float* xml = xo + 3 * 16 * dv;                              // [3][16][2]
        if (warp > 0) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = g + 8 * half;
                float* dst = xo + ((warp - 1) * 16 + r) * dv + 2 * t4;
#pragma unroll
                for (int i = 0; i < MAXDV8; ++i)
                    if (i < dv8) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o_acc[i][2 * half], o_acc[i][2 * half + 1]);
                if (t4 == 0) {
                    xml[((warp - 1) * 16 + r) * 2] = m_run[half];
                    xml[((warp - 1) * 16 + r) * 2 + 1] = l_run[half];
                }
            }
        }
        __syncthreads();
        if (warp > 0) return;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            float mx = m_run[half];
            for (int w = 0; w < 3; ++w) mx = fmaxf(mx, xml[(w * 16 + r) * 2]);
            const float base = mx == -INFINITY ? 0.f : mx;
            const float mine = exp2f(m_run[half] - base);
            float wgt[3];
            float l = l_run[half] * mine;
            for (int w = 0; w < 3; ++w) {
                wgt[w] = exp2f(xml[(w * 16 + r) * 2] - base);
                l = fmaf(wgt[w], xml[(w * 16 + r) * 2 + 1], l);
            }
#pragma unroll
            for (int i = 0; i < MAXDV8; ++i) {
                if (i < dv8) {
                    float v0 = o_acc[i][2 * half] * mine, v1 = o_acc[i][2 * half + 1] * mine;
                    for (int w = 0; w < 3; ++w) {
                        const float2 o = *reinterpret_cast<const float2*>(xo + (w * 16 + r) * dv + i * 8 + 2 * t4);
                        v0 = fmaf(wgt[w], o.x, v0);
                        v1 = fmaf(wgt[w], o.y, v1);
                    }
                    o_acc[i][2 * half] = v0;
                    o_acc[i][2 * half + 1] = v1;
                }
            }
            m_run[half] = mx;
            l_run[half] = l;
        }
    }

    if (splits == 1) {
        const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r_b : r_a;
            if (r >= n_rows) continue;
            const int row = row0 + r;
            __nv_bfloat16* dst = out + ((long long)(q_first + row / heads) * heads + row % heads) * dv + 2 * t4;
            const float inv = half ? inv_b : inv_a;
#pragma unroll
            for (int i = 0; i < MAXDV8; ++i)
                if (i < dv8)
                    *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) =
                        __floats2bfloat162_rn(o_acc[i][2 * half] * inv, o_acc[i][2 * half + 1] * inv);
        }
        return;
    }
    // a slice: its unnormalised sums with its maximum (log2 units) and its sum of weights
    const long long slot = ((long long)blockIdx.x * splits + split) * BM;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r_b : r_a;
        if (r >= n_rows) continue;
        float* dst = part_o + (slot + r) * dv + 2 * t4;
#pragma unroll
        for (int i = 0; i < MAXDV8; ++i)
            if (i < dv8) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o_acc[i][2 * half], o_acc[i][2 * half + 1]);
        if (t4 == 0) {
            part_ml[(slot + r) * 2] = m_run[half];
            part_ml[(slot + r) * 2 + 1] = l_run[half];
        }
    }
}

// out[row] = sum_s w_s O_s / sum_s w_s l_s, w_s = 2^(m_s - max m), over a tile's slices in order.
// A CTA per (tile, row): the slices' weights once, in shared memory, then a thread per column.
constexpr int MAX_SPLITS = 64;
template <bool SMALL>
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q, int n_entries,
                         int heads, int dv, int splits) {
    constexpr int BM = SMALL ? 16 : 64;
    __shared__ float wgt[MAX_SPLITS];
    __shared__ float inv_den;
    pdl_launch_dependents();
    int entry, row0;
    if (!find_tile(blockIdx.x, cu_q, n_entries, heads, BM, SMALL, entry, row0)) return;
    const int q_first = cu_q[entry], rows = (cu_q[entry + 1] - q_first) * heads;
    const int r = blockIdx.y;
    if (row0 + r >= rows) return;
    pdl_wait();
    const long long first = ((long long)blockIdx.x * splits) * BM + r;       // slice s: first + s * BM
    if (threadIdx.x < 32) {
        float mx = -INFINITY;
        for (int s = threadIdx.x; s < splits; s += 32) mx = fmaxf(mx, part_ml[(first + (long long)s * BM) * 2]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int s = threadIdx.x; s < splits; s += 32) {
            const float m = part_ml[(first + (long long)s * BM) * 2];
            const float w = m == -INFINITY ? 0.f : exp2f(m - mx);
            wgt[s] = w;
            den = fmaf(w, part_ml[(first + (long long)s * BM) * 2 + 1], den);
        }
        den = warp_sum(den);
        if (threadIdx.x == 0) inv_den = den > 0.f ? 1.f / den : 0.f;
    }
    __syncthreads();
    const int row = row0 + r;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float num = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float w = wgt[s];
            const float v = part_o[(first + (long long)s * BM) * dv + c];     // (an empty slice left nothing here)
            num += w != 0.f ? w * v : 0.f;
        }
        out[((long long)q_first * heads + row) * dv + c] = __float2bfloat16_rn(num * inv_den);
    }
}

template <bool SMALL, int MAXDK16, int MAXDV8>
int launch(const __nv_bfloat16* q, __nv_bfloat16* out, float* part_o, float* part_ml, const __nv_bfloat16* pool,
           const int* cu_q, const int* kv_len, const int* block_table, int max_blocks, int num_pages, int page_size,
           int n_entries, int tiles, int splits, int heads, int dk, int dv, float scale, int* err, cudaStream_t st) {
    constexpr int BM = SMALL ? 16 : 64;
    constexpr int KT = KeyTile<SMALL>::value;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    if ((1 << page_shift) != page_size) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(BM + 2 * KT) * (dk + 8) * sizeof(__nv_bfloat16);
    auto kern = latent_attn_mma_kernel<SMALL, MAXDK16, MAXDV8>;
    static bool attr_set = false;                    // (one flag per instantiation)
    if (smem > 48 * 1024 && !attr_set) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set = true;
    }
    int rc = crane_launch(kern, dim3(tiles, splits), dim3(128), smem, st, q, out, part_o, part_ml, pool, cu_q,
                          kv_len, block_table, max_blocks, num_pages, page_shift, n_entries, heads, dk, dv, scale, err);
    if (rc != 0 || splits == 1) return rc;
    return crane_launch(latent_attn_merge_kernel<SMALL>, dim3(tiles, BM), dim3(128), 0, st, (const float*)part_o,
                        (const float*)part_ml, out, cu_q, n_entries, heads, dv, splits);
}

}  // namespace

// 1 if the tensor-core kernel takes these widths.
CRANE_API int crane_latent_attention_mma_supports(int dk, int dv) {
    return dk > 0 && dv > 0 && dk % 16 == 0 && dv % 8 == 0 && dv <= dk && dk <= 256 && dv <= 192 ? 1 : 0;
}

// `small` 1: the entries of one token or of at most 16 rows (tokens x heads), in tiles of 16 rows; 0: the
// others, in tiles of 64.  Pages of a power of two.  `tiles`: at least the number of such tiles.  splits > 1 needs part_o [tiles * splits * rows per
// tile * dv] and part_ml [tiles * splits * rows per tile * 2] floats.
CRANE_API int crane_latent_attention_mma(const void* q, void* out, float* part_o, float* part_ml, const void* pool,
                                         const int* cu_q, const int* kv_len, const int* block_table,
                                         int max_blocks, int num_pages, int page_size, int n_entries, int tiles,
                                         int splits, int small, int heads, int dk, int dv, float scale, int* err,
                                         cudaStream_t st) {
    if (tiles <= 0 || n_entries <= 0) return 0;
    if (!crane_latent_attention_mma_supports(dk, dv) || splits < 1 || splits > MAX_SPLITS ||
        (splits > 1 && (part_o == nullptr || part_ml == nullptr)))
        return (int)cudaErrorInvalidValue;
    const auto* qb = (const __nv_bfloat16*)q;
    auto* ob = (__nv_bfloat16*)out;
    const auto* pb = (const __nv_bfloat16*)pool;
#define CRANE_LATENT_LAUNCH(W, A, B)                                                                          \
    return launch<W, A, B>(qb, ob, part_o, part_ml, pb, cu_q, kv_len, block_table, max_blocks, num_pages,     \
                           page_size, n_entries, tiles, splits, heads, dk, dv, scale, err, st)
    const bool narrow = dk <= 128 && dv <= 128;
    if (small) {
        if (narrow) CRANE_LATENT_LAUNCH(true, 8, 16);
        CRANE_LATENT_LAUNCH(true, 16, 24);
    }
    if (narrow) CRANE_LATENT_LAUNCH(false, 8, 16);
    CRANE_LATENT_LAUNCH(false, 16, 24);
#undef CRANE_LATENT_LAUNCH
}
