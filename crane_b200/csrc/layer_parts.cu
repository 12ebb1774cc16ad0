// Memory-bound kernels of layers that are not Hunyuan Dense's: a token embedding with a hashed
// bigram table added, the sum of a parallel block's two branches with the depth-weighted average
// of all earlier layers' results and the (one or two) layer norms that read the new stream, and
// the xIELU activation.  All arithmetic in 32-bit; T is the storage type of activations and
// weights (float or bf16).  The residual stream and the history of layer results are float.
#include "common.cuh"

// ------------------------------------------------------ embedding + bigram
// x[t] = table[tok] + bigram[(prev * mul_prev + tok * mul_cur) mod buckets]; the first token of a
// sequence (position 0) takes row `buckets`.  The token before a portion's first one is the
// request's state: last_token[slot], read and then replaced (by the entry's last token) by the
// CTA of the entry's first row alone.  Rows of no entry (tok_entry < 0) get the plain embedding
// and touch no state.  A token id <= -2 names row (-id - 2) of `deferred`.
template <typename T>
__global__ void __launch_bounds__(256)
embed_bigram_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                    const T* __restrict__ bigram, float* __restrict__ x, int hidden, int vocab,
                    int buckets, long long mul_prev, long long mul_cur,
                    const int* __restrict__ positions, const int* __restrict__ tok_entry,
                    const int* __restrict__ cu_q, const int* __restrict__ slots,
                    int* __restrict__ last_token, int n_slots, const int* __restrict__ deferred,
                    int n_deferred, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    auto resolve = [&](int tok) {
        if (tok <= -2 && deferred != nullptr && -tok - 2 < n_deferred) tok = deferred[-tok - 2];
        if (tok < 0 || tok >= vocab) {
            if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_TOKEN_RANGE);
            tok = 0;
        }
        return tok;
    };
    const int tok = resolve(tokens[t]);
    const int e = tok_entry[t];
    const T* src = table + (long long)tok * hidden;
    float* dst = x + (long long)t * hidden;
    if (e < 0 || bigram == nullptr) {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]);
        return;
    }
    const int first = cu_q[e];
    int slot = slots[e];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_SLOT_RANGE);
        slot = 0;
    }
    int row = buckets;
    if (positions[t] > 0) {
        const int prev = t > first ? resolve(tokens[t - 1]) : last_token[slot];
        long long hsh = ((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
        if (hsh < 0) hsh += buckets;
        row = (int)hsh;
    }
    if (t == first) {
        __syncthreads();                  // every thread has read the state
        if (threadIdx.x == 0) last_token[slot] = resolve(tokens[cu_q[e + 1] - 1]);
    }
    const T* bg = bigram + (long long)row * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]) + to_f32(bg[c]);
}

// ------------------------------ branch sum + depth-weighted average + layer norm(s)
// X_new = x + (a + f)  (the branches of a parallel block; either may be absent)
// hist[n_hist - 1] = X_new;  x = sum_j dwa[j] * hist[j], j = 0 .. n_hist - 1 in order (dwa null: x = X_new)
// out1 = LN(x; w1, b1), out2 = LN(x; w2, b2) (out2 null: one norm), LN(x) = (x - mean) / sqrt(var + eps) * w + b
// with var the mean of the squared deviations.
// rows == nullptr: row r = blockIdx.x, x and hist are updated.  rows != nullptr: row = rows[r] is
// read, nothing but out1 / out2 [r] is written (the final norm over the wanted rows).
template <typename T>
__global__ void __launch_bounds__(1024)
combine_layernorm_kernel(float* __restrict__ x, float* __restrict__ hist, long long hist_stride,
                         int n_hist, GemmOut<T> a, int has_a, GemmOut<T> f, int has_f,
                         const float* __restrict__ dwa, const int* __restrict__ rows,
                         const float* __restrict__ w1, const float* __restrict__ b1,
                         T* __restrict__ out1, const float* __restrict__ w2,
                         const float* __restrict__ b2, T* __restrict__ out2, int hidden, float eps) {
    extern __shared__ float vals[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int row = rows ? rows[r] : r;
    const long long base = (long long)row * hidden;
    float sum = 0.f;
    // four columns per thread and pass, so that the loads of the earlier results (one per history
    // entry and column, independent of one another) are in flight together
    for (int c0 = threadIdx.x * 4; c0 < hidden; c0 += blockDim.x * 4) {
        const int nc = min(4, hidden - c0);
        float xn[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            xn[k] = 0.f;
            if (k < nc) {
                xn[k] = x[base + c0 + k];
                if (has_a || has_f) {
                    float branches = has_a ? a.load(base + c0 + k) : 0.f;
                    if (has_f) branches = has_a ? branches + f.load(base + c0 + k) : f.load(base + c0 + k);
                    xn[k] += branches;
                }
            }
        }
        if (dwa != nullptr) {
#pragma unroll 4
            for (int j = 0; j + 1 < n_hist; ++j) {
                const float wj = dwa[j];
                const float* hp = hist + j * hist_stride + base + c0;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < nc) acc[k] = fmaf(wj, hp[k], acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (k >= nc) break;
            const int c = c0 + k;
            const float val = dwa != nullptr ? fmaf(dwa[n_hist - 1], xn[k], acc[k]) : xn[k];
            if (rows == nullptr) {
                if (hist != nullptr) hist[(long long)(n_hist - 1) * hist_stride + base + c] = xn[k];
                x[base + c] = val;
            }
            vals[c] = val;
            sum += val;
        }
    }
    const float mean = block_sum(sum, scratch) / (float)hidden;
    float sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float dlt = vals[c] - mean;
        sq += dlt * dlt;
    }
    const float rstd = 1.f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps);
    const long long ob = (long long)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float nv = (vals[c] - mean) * rstd;
        if (out1 != nullptr) out1[ob + c] = from_f32<T>(nv * w1[c] + b1[c]);
        if (out2 != nullptr) out2[ob + c] = from_f32<T>(nv * w2[c] + b2[c]);
    }
}

// ------------------------------------------------------------------ xIELU
// z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void xielu_kernel(GemmOut<T> src, T* __restrict__ out, long long n,
                             const float* __restrict__ pq) {
    pdl_launch_dependents();
    const float ap = softplus_f(pq[0]), aq = 0.5f + softplus_f(pq[1]);
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = src.load(i);
    const float y = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
    out[i] = from_f32<T>(y);
}

// the same for a whole bf16 tensor, eight elements (16 bytes) per thread
__global__ void xielu_bf16x8_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ out,
                                    long long n8, const float* __restrict__ pq) {
    pdl_launch_dependents();
    const float ap = softplus_f(pq[0]), aq = 0.5f + softplus_f(pq[1]);
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    uint4 raw = reinterpret_cast<const uint4*>(src)[i];
    __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 z = __bfloat1622float2(v[k]);
        z.x = z.x > 0.f ? fmaf(ap * z.x, z.x, 0.5f * z.x) : fmaf(aq, expm1f(z.x) - z.x, 0.5f * z.x);
        z.y = z.y > 0.f ? fmaf(ap * z.y, z.y, 0.5f * z.y) : fmaf(aq, expm1f(z.y) - z.y, 0.5f * z.y);
        v[k] = __floats2bfloat162_rn(z.x, z.y);
    }
    reinterpret_cast<uint4*>(out)[i] = raw;
}

CRANE_API int crane_embed_bigram(int dtype, const int* tokens, const void* table, const void* bigram,
                                 float* x, int n_tokens, int hidden, int vocab, int buckets,
                                 long long mul_prev, long long mul_cur, const int* positions,
                                 const int* tok_entry, const int* cu_q, const int* slots,
                                 int* last_token, int n_slots, const int* deferred, int n_deferred,
                                 int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (bigram != nullptr && buckets <= 0) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, return crane_launch(embed_bigram_kernel<T>, dim3(n_tokens), dim3(256), 0, st, tokens,
                                          (const T*)table, (const T*)bigram, x, hidden, vocab, buckets,
                                          mul_prev, mul_cur, positions, tok_entry, cu_q, slots, last_token,
                                          n_slots, deferred, n_deferred, err));
}

CRANE_API int crane_combine_layernorm(int dtype, float* x, float* hist, long long hist_stride, int n_hist,
                                      const void* a, const float* a_parts, int a_n, long long a_stride,
                                      const void* f, const float* f_parts, int f_n, long long f_stride,
                                      const float* dwa, const int* rows, const float* w1, const float* b1,
                                      void* out1, const float* w2, const float* b2, void* out2,
                                      int n_rows, int hidden, float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int has_a = (a != nullptr || a_parts != nullptr) ? 1 : 0;
    const int has_f = (f != nullptr || f_parts != nullptr) ? 1 : 0;
    DISPATCH_T(dtype, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(combine_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
        GemmOut<T> ga{(const T*)a, a_parts, a_n, a_stride};
        GemmOut<T> gf{(const T*)f, f_parts, f_n, f_stride};
        // four columns per thread in one pass where the row allows it (few rows: a step of decoded
        // tokens, where a row's chain of loads is all there is to wait for)
        int threads = (hidden / 4 + 31) / 32 * 32;
        threads = threads < 128 ? 128 : threads > 1024 ? 1024 : threads;
        if (n_rows > 512 && threads > 256) threads = 256;
        return crane_launch(combine_layernorm_kernel<T>, dim3(n_rows), dim3(threads), smem, st, x, hist,
                            hist_stride, n_hist, ga, has_a, gf, has_f, dwa, rows, w1, b1, (T*)out1, w2, b2,
                            (T*)out2, hidden, eps);
    });
}

CRANE_API int crane_xielu(int dtype, const void* up, const float* up_parts, int n_parts,
                          long long part_stride, void* out, long long n, const float* pq,
                          cudaStream_t st) {
    if (n <= 0) return 0;
    if (dtype == 1 && up != nullptr && n % 8 == 0 && ((uintptr_t)up | (uintptr_t)out) % 16 == 0)
        return crane_launch(xielu_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st,
                            (const __nv_bfloat16*)up, (__nv_bfloat16*)out, n / 8, pq);
    DISPATCH_T(dtype, {
        GemmOut<T> src{(const T*)up, up_parts, n_parts, part_stride};
        return crane_launch(xielu_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, src,
                            (T*)out, n, pq);
    });
}
