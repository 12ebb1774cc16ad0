// Latent attention: keys and values of all heads are up-projections of one cached latent vector
// c [rank] per position, plus one rotated key part kr [rot] shared by all heads.  With
// k_h = U_h c and v_h = V_h c the score of head h is q_h . k_h + qr_h . kr = (U_h^T q_h) . c + qr_h . kr
// and its output V_h (sum_j p_j c_j): attention runs in the latent space as one shared key/value
// "head" of width rank + rot (value: the leading rank columns of the same rows), between two small
// per-head products.  The kernels here are those products and the step that fills the cache:
//
// latent_prep   per token: c = RMSNorm(first rank columns of the down projection) * w and the rotated
//               last rot columns go to the token's cache row [rank + rot]; the rotated part of every
//               query head goes to columns rank.. of the absorbed query [token, head, rank + rot].
// head_linear   out[t, h, :] = W_h x[t, h, :] for every head (U_h^T on the unrotated query part; V_h on
//               the attention's latent output, there times sigmoid(gate)): on the tensor cores in
//               bfloat16 (widths that the MMA tiles take), else on the FP32 cores.
//
// Rotation: interleaved pairs (2i, 2i + 1) of the leading rot_dims elements of the rotated part,
// (u, v) -> (u cos - v sin, v cos + u sin); the tables hold cos and sin already scaled.
// All arithmetic in 32-bit; T is the storage type (float or bf16).
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(GemmOut<T> proj, int cols, int q_off, int dkv_off, int heads, int dim, int rot,
                   int rank, int rot_dims, const float* __restrict__ cos_tab,
                   const float* __restrict__ sin_tab, int n_positions,
                   const int* __restrict__ positions, const int* __restrict__ tok_entry,
                   const int* __restrict__ block_table, int max_blocks, int num_pages, int page_size,
                   T* __restrict__ pool, const float* __restrict__ norm_w, float eps,
                   T* __restrict__ q_abs, int* err) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int e = tok_entry[t];
    if (e < 0) return;                                  // a row that pads the step
    int pos = positions[t];
    if (pos < 0 || pos >= n_positions) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_POSITION_RANGE);
        pos = 0;
    }
    const long long prow = (long long)t * cols;
    const int half = rot_dims >> 1, pairs = rot >> 1, width = rank + rot;
    const float* cs = cos_tab + (long long)pos * half;
    const float* sn = sin_tab + (long long)pos * half;
    // the rotated part of every query head
    for (int i = threadIdx.x; i < heads * pairs; i += blockDim.x) {
        const int h = i / pairs, p = i % pairs;
        const long long src = prow + q_off + (long long)h * (dim + rot) + dim + 2 * p;
        float u = proj.load(src), v = proj.load(src + 1);
        if (p < half) {
            const float c = cs[p], s = sn[p];
            const float u2 = u * c - v * s, v2 = v * c + u * s;
            u = u2;
            v = v2;
        }
        T* dst = q_abs + ((long long)t * heads + h) * width + rank + 2 * p;
        dst[0] = from_f32<T>(u);
        dst[1] = from_f32<T>(v);
    }
    if (dkv_off < 0) return;                            // the layer reads another layer's cache
    const int page = block_table[(long long)e * max_blocks + pos / page_size];
    const bool ok = page >= 0 && page < num_pages;
    if (!ok && threadIdx.x == 0) atomicOr(err, CRANE_ERR_PAGE_RANGE);
    T* crow = pool + ((long long)(ok ? page : 0) * page_size + pos % page_size) * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = proj.load(prow + dkv_off + c);
        ss += v * v;
    }
    const float rstd = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    if (!ok) return;
    for (int c = threadIdx.x; c < rank; c += blockDim.x)
        crow[c] = from_f32<T>(proj.load(prow + dkv_off + c) * rstd * norm_w[c]);
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const long long src = prow + dkv_off + rank + 2 * p;
        float u = proj.load(src), v = proj.load(src + 1);
        if (p < half) {
            const float c = cs[p], s = sn[p];
            const float u2 = u * c - v * s, v2 = v * c + u * s;
            u = u2;
            v = v2;
        }
        crow[rank + 2 * p] = from_f32<T>(u);
        crow[rank + 2 * p + 1] = from_f32<T>(v);
    }
}

// out[t, h, o] = sum_i w[h][i][o] * x[t, x_off + h * x_head + i]  (i in order 0 .. n_in - 1), then
// times sigmoid(gate[t, g_off + h * n_out + o]) if a gate is given.  x and gate are columns of
// one product's result (row pitch x_cols / g_cols).  A CTA takes TT tokens of one head.
constexpr int HL_TT = 16;
constexpr int HL_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(GemmOut<T> x, int x_cols, int x_off, int x_head, const T* __restrict__ w, int n_in,
                   int n_out, GemmOut<T> gate, int has_gate, int g_cols, int g_off,
                   const int* __restrict__ tok_entry, T* __restrict__ out, int out_pitch,
                   int out_head, int n_tokens, int heads) {
    extern __shared__ float xs[];                       // [HL_TT][n_in]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.x * HL_TT;
    const int nt = min(HL_TT, n_tokens - t0);
    for (int i = threadIdx.x; i < nt * n_in; i += blockDim.x) {
        const int tt = i / n_in, c = i % n_in;
        xs[tt * n_in + c] = x.load((long long)(t0 + tt) * x_cols + x_off + (long long)h * x_head + c);
    }
    __syncthreads();
    const T* wh = w + (long long)h * n_in * n_out;
    for (int o = threadIdx.x; o < n_out; o += blockDim.x) {
        float acc[HL_TT];
#pragma unroll
        for (int tt = 0; tt < HL_TT; ++tt) acc[tt] = 0.f;
        for (int i = 0; i < n_in; ++i) {
            const float wv = to_f32(wh[(long long)i * n_out + o]);
#pragma unroll
            for (int tt = 0; tt < HL_TT; ++tt) acc[tt] = fmaf(wv, xs[tt * n_in + i], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_TT; ++tt) {
            if (tt >= nt) break;
            const int t = t0 + tt;
            if (tok_entry != nullptr && tok_entry[t] < 0) continue;
            float v = to_f32(from_f32<T>(acc[tt]));
            if (has_gate) {
                const float g = gate.load((long long)t * g_cols + g_off + (long long)h * n_out + o);
                v *= 1.f / (1.f + expf(-g));
            }
            out[(long long)t * out_pitch + (long long)h * out_head + o] = from_f32<T>(v);
        }
    }
}

// ---- the same product on the tensor cores (bf16, warp-level MMA) -------------------------------
// A CTA takes 64 tokens of one head: the head's matrix [n_in][n_out] and the tokens' inputs come
// into shared memory by cp.async, each of four warps multiplies 16 tokens by the whole matrix
// (B fragments by transposed ldmatrix, since the matrix is stored inputs-major), rounds to bf16,
// applies the gate and writes.  Taken for bf16 with n_in a multiple of 16 and n_out of 8, both at
// most 256, and 16-byte aligned rows; operands left as partial sums are added up on the way in.
__device__ __forceinline__ void hl_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void hl_ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void hl_cp16(void* smem, const void* gmem, bool valid) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(gmem), "r"(n));
}

constexpr int HM_TT = 64;
template <int MAXK16, int MAXN8, bool FEW>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(GemmOut<__nv_bfloat16> x, int x_cols, int x_off, int x_head,
                       const __nv_bfloat16* __restrict__ w, int n_in, int n_out,
                       GemmOut<__nv_bfloat16> gate, int has_gate, int g_cols, int g_off,
                       const int* __restrict__ tok_entry, __nv_bfloat16* __restrict__ out, int out_pitch,
                       int out_head, int n_tokens) {
    extern __shared__ __align__(16) unsigned char hl_smem[];
    const int lda = n_in + 8, ldw = n_out + 8;
    __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(hl_smem);      // [64][lda]
    __nv_bfloat16* w_s = a_s + HM_TT * lda;                               // [n_in][ldw]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.y, t0 = blockIdx.x * HM_TT;
    pdl_launch_dependents();
    // the head's matrix depends on no earlier kernel
    const __nv_bfloat16* wh = w + (long long)h * n_in * n_out;
    {
        const int n16w = (n_out + 15) >> 4;
        const int zper = FEW ? (n16w + (int)gridDim.z - 1) / (int)gridDim.z : n16w;
        const int c_lo = FEW ? (int)blockIdx.z * zper * 2 : 0;
        const int c_hi = min(n_out >> 3, c_lo + zper * 2);
        for (int r = warp; r < n_in; r += 4)
            for (int c = c_lo + lane; c < c_hi; c += 32) hl_cp16(w_s + r * ldw + c * 8, wh + (long long)r * n_out + c * 8, true);
    }
    pdl_wait();
    // At most 16 tokens in the tile (a decode step): the four warps share the one block of 16 rows and
    // take a quarter of the output columns each, instead of a block of rows each.
    constexpr bool few = FEW;                                       // (the launch has 16 tokens at most)
    const int wrow = few ? 0 : warp * 16;
    const int n16 = (n_out + 15) >> 4;                              // pairs of 8 output columns
    // (and the few-token form spreads the columns over gridDim.z CTAs first, each of which fetches its
    // columns of the matrix alone)
    const int cta_per = few ? (n16 + (int)gridDim.z - 1) / (int)gridDim.z : n16;
    const int cta_lo = few ? (int)blockIdx.z * cta_per : 0, cta_hi = min(n16, cta_lo + cta_per);
    const int per = few ? (cta_hi - cta_lo + 3) >> 2 : n16;
    const int n2_lo = few ? cta_lo + warp * per : 0, n2_hi = few ? min(cta_hi, n2_lo + per) : n16;
    for (int r = warp; r < (few ? 16 : HM_TT); r += 4) {
        const bool ok = t0 + r < n_tokens;
        const long long at = ok ? (long long)(t0 + r) * x_cols + x_off + (long long)h * x_head : 0;
        if (x.parts == nullptr) {
            for (int c = lane; c < (n_in >> 3); c += 32) hl_cp16(a_s + r * lda + c * 8, x.whole + at + c * 8, ok);
        } else {                                        // partial sums: added up and rounded here
            for (int c = lane; c < (n_in >> 1); c += 32) {
                const float2 v = ok ? x.load2(at + 2 * c) : make_float2(0.f, 0.f);
                *reinterpret_cast<__nv_bfloat162*>(a_s + r * lda + 2 * c) = __floats2bfloat162_rn(v.x, v.y);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float acc[MAXN8][4];
#pragma unroll
    for (int i = 0; i < MAXN8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int k16 = n_in >> 4, n8 = n_out >> 3;
#pragma unroll 1
    for (int ks = 0; ks < k16; ++ks) {
        uint32_t a0, a1, a2, a3;
        hl_ldsm_x4(a0, a1, a2, a3, a_s + (wrow + (lane & 15)) * lda + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < MAXN8 / 2; ++n2) {
            if (n2 >= n2_lo && n2 < n2_hi) {
                uint32_t b0, b1, b2, b3;
                hl_ldsm_x4_t(b0, b1, b2, b3, w_s + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldw + n2 * 16 + (lane >> 4) * 8);
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(acc[2 * n2][0]), "+f"(acc[2 * n2][1]), "+f"(acc[2 * n2][2]), "+f"(acc[2 * n2][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
                if (2 * n2 + 1 < n8)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(acc[2 * n2 + 1][0]), "+f"(acc[2 * n2 + 1][1]), "+f"(acc[2 * n2 + 1][2]), "+f"(acc[2 * n2 + 1][3])
                                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b2), "r"(b3));
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int t = t0 + wrow + g + 8 * half;
        if (t >= n_tokens || (tok_entry != nullptr && tok_entry[t] < 0)) continue;
        __nv_bfloat16* dst = out + (long long)t * out_pitch + (long long)h * out_head + 2 * t4;
        const long long gp = (long long)t * g_cols + g_off + (long long)h * n_out + 2 * t4;
#pragma unroll
        for (int i = 0; i < MAXN8; ++i) {
            if (i < n8 && (i >> 1) >= n2_lo && (i >> 1) < n2_hi) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[i][2 * half], acc[i][2 * half + 1]);
                if (has_gate) {
                    const float2 gv = gate.load2(gp + i * 8);
                    const float2 f = __bfloat1622float2(v);
                    v = __floats2bfloat162_rn(f.x / (1.f + expf(-gv.x)), f.y / (1.f + expf(-gv.y)));
                }
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = v;
            }
        }
    }
}

}  // namespace

CRANE_API int crane_latent_prep(int dtype, const void* proj, const float* proj_parts, int n_parts,
                                long long part_stride, int cols, int q_off, int dkv_off, int heads,
                                int dim, int rot, int rank, int rot_dims, const float* cos_tab,
                                const float* sin_tab, int n_positions, const int* positions,
                                const int* tok_entry, const int* block_table, int max_blocks,
                                int num_pages, int page_size, void* pool, const float* norm_w, float eps,
                                void* q_abs, int n_tokens, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if ((rot & 1) || (rot_dims & 1) || rot_dims > rot || rot_dims < 0) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> p{(const T*)proj, proj_parts, n_parts, part_stride};
        return crane_launch(latent_prep_kernel<T>, dim3(n_tokens), dim3(128), 0, st, p, cols, q_off, dkv_off,
                            heads, dim, rot, rank, rot_dims, cos_tab, sin_tab, n_positions, positions,
                            tok_entry, block_table, max_blocks, num_pages, page_size, (T*)pool, norm_w, eps,
                            (T*)q_abs, err);
    });
}

CRANE_API int crane_head_linear(int dtype, const void* x, const float* x_parts, int x_n, long long x_stride,
                                int x_cols, int x_off, int x_head, const void* w, int n_in, int n_out,
                                const void* gate, const float* g_parts, int g_n, long long g_stride,
                                int g_cols, int g_off, const int* tok_entry, void* out, int out_pitch,
                                int out_head, int n_tokens, int heads, cudaStream_t st) {
    if (n_tokens <= 0 || heads <= 0) return 0;
    const bool aligned = x_cols % 8 == 0 && x_off % 8 == 0 && x_head % 8 == 0 && out_pitch % 2 == 0 &&
                         out_head % 2 == 0 && g_cols % 2 == 0 && g_off % 2 == 0 &&
                         ((uintptr_t)x | (uintptr_t)w) % 16 == 0 && ((uintptr_t)out | (uintptr_t)gate) % 4 == 0;
    if (dtype == 1 && aligned && n_in % 16 == 0 && n_out % 8 == 0 && n_in <= 256 && n_out <= 256) {
        const size_t sm = ((size_t)HM_TT * (n_in + 8) + (size_t)n_in * (n_out + 8)) * sizeof(__nv_bfloat16);
        // (the column blocks are unrolled: an instantiation per bound keeps the code of the common widths short)
        const bool few_tokens = n_tokens <= 16;
        const int n8 = n_out >> 3;
        auto kern = n8 <= 16 ? (few_tokens ? head_linear_mma_kernel<16, 16, true> : head_linear_mma_kernel<16, 16, false>)
                  : n8 <= 24 ? (few_tokens ? head_linear_mma_kernel<16, 24, true> : head_linear_mma_kernel<16, 24, false>)
                             : (few_tokens ? head_linear_mma_kernel<16, 32, true> : head_linear_mma_kernel<16, 32, false>);
        static bool attr_set = false;
        if (!attr_set) {
            const int most = 200 * 1024;
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 24, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 24, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            cudaFuncSetAttribute(head_linear_mma_kernel<16, 32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
            attr_set = true;
        }
        GemmOut<__nv_bfloat16> gx{(const __nv_bfloat16*)x, x_parts, x_n, x_stride};
        GemmOut<__nv_bfloat16> gg{(const __nv_bfloat16*)gate, g_parts, g_n, g_stride};
        const int zs = n_tokens <= 16 ? ((n_out + 15) / 16 < 4 ? (n_out + 15) / 16 : 4) : 1;
        return crane_launch(kern, dim3((n_tokens + HM_TT - 1) / HM_TT, heads, zs), dim3(128), sm, st, gx, x_cols, x_off,
                            x_head, (const __nv_bfloat16*)w, n_in, n_out, gg,
                            (gate != nullptr || g_parts != nullptr) ? 1 : 0, g_cols, g_off, tok_entry,
                            (__nv_bfloat16*)out, out_pitch, out_head, n_tokens);
    }
    const size_t smem = (size_t)HL_TT * n_in * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int has_gate = (gate != nullptr || g_parts != nullptr) ? 1 : 0;
    DISPATCH_T(dtype, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        GemmOut<T> gx{(const T*)x, x_parts, x_n, x_stride};
        GemmOut<T> gg{(const T*)gate, g_parts, g_n, g_stride};
        return crane_launch(head_linear_kernel<T>, dim3((n_tokens + HL_TT - 1) / HL_TT, heads),
                            dim3(HL_THREADS), smem, st, gx, x_cols, x_off, x_head, (const T*)w, n_in, n_out, gg,
                            has_gate, g_cols, g_off, tok_entry, (T*)out, out_pitch, out_head, n_tokens, heads);
    });
}
