// Memory-bound kernels around the residual stream of layers that norm a sublayer's result before
// they add it: a token embedding with a sinusoidal position vector added, the vector (and the kept
// embedding output) added where a pass over repeated layers begins, the addition of a normed
// sublayer result fused with the norm that reads the stream next, the gate of a per-layer token
// input, and the activations of plain and routed feed-forwards.  All arithmetic in 32-bit (angles
// in 64-bit); T is the storage type of activations and weights (float or bf16).  The stream is float.
#include "common.cuh"

namespace {

__device__ __forceinline__ int resolve_token(int tok, int vocab, const int* deferred, int n_deferred, int* err) {
    if (tok <= -2 && deferred != nullptr && -tok - 2 < n_deferred) tok = deferred[-tok - 2];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, CRANE_ERR_TOKEN_RANGE);
        tok = 0;
    }
    return tok;
}

// ------------------------------------------------------ embedding + sinusoid
// x[t][2i] = table[tok][2i] + sin(p f_i), x[t][2i + 1] = table[tok][2i + 1] + cos(p f_i); `freq` holds
// the f_i as doubles (the host forms base^(-2i / hidden) in 64-bit).  The angle is formed and brought
// into [-pi, pi] in 64-bit, its sine and cosine are taken in 32-bit from there.  `keep`: a second
// copy of the rows (the embedding output, for a model that adds it again later).
template <typename T>
__global__ void __launch_bounds__(256)
embed_sinusoid_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                      const T* __restrict__ table, const double* __restrict__ freq,
                      float* __restrict__ x, float* __restrict__ keep, int hidden, int vocab,
                      const int* __restrict__ deferred, int n_deferred, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = resolve_token(tokens[t], vocab, deferred, n_deferred, err);
    const double p = (double)positions[t];
    const T* src = table + (long long)tok * hidden;
    const long long base = (long long)t * hidden;
    constexpr double TWO_PI = 6.283185307179586476925286766559;
    for (int i = threadIdx.x; 2 * i < hidden; i += blockDim.x) {
        double a = p * freq[i];
        a -= TWO_PI * rint(a / TWO_PI);
        float s, c;
        sincosf((float)a, &s, &c);
        const float v0 = to_f32(src[2 * i]) + s;
        x[base + 2 * i] = v0;
        if (keep != nullptr) keep[base + 2 * i] = v0;
        if (2 * i + 1 < hidden) {
            const float v1 = to_f32(src[2 * i + 1]) + c;
            x[base + 2 * i + 1] = v1;
            if (keep != nullptr) keep[base + 2 * i + 1] = v1;
        }
    }
}

// ------------------------------------------------------ where a pass begins
// x += kept (if given) + vec
__global__ void __launch_bounds__(256)
stream_enter_kernel(float* __restrict__ x, const float* __restrict__ kept, const float* __restrict__ vec,
                    long long n, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (kept != nullptr) v += kept[i];
        x[i] = v + vec[i % hidden];
    }
}

// ------------------------------------------------------ x += norm(delta); out = norm(x)
// y = delta / sqrt(mean(delta^2) + eps) * wd;  x += y;  out = x / sqrt(mean(x^2) + eps) * wo (if out);
// raw = x in T (if raw).  The weights are what the norms multiply by (an offset is folded in by the host).
// One CTA per row; the row lives in shared memory between the passes.
template <typename T>
__global__ void __launch_bounds__(1024)
add_normed_norm_kernel(float* __restrict__ x, GemmOut<T> delta, const float* __restrict__ wd,
                       const float* __restrict__ wo, T* __restrict__ out, T* __restrict__ raw,
                       int hidden, float eps_d, float eps_o) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const long long base = (long long)blockIdx.x * hidden;
    float ss = 0.f;
    // (rows of a multiple of 4 columns go four columns a thread and pass; `hidden` and the tensors'
    // alignment are the same for every row, so the branch is uniform)
    const bool quad = hidden % 4 == 0 && delta.parts == nullptr && ((uintptr_t)delta.whole % 8) == 0 &&
                      ((uintptr_t)x | (uintptr_t)wd | (uintptr_t)wo) % 16 == 0 && ((uintptr_t)out | (uintptr_t)raw) % 8 == 0;
    if (quad) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float2 a = ld2(delta.whole + base + c), b = ld2(delta.whole + base + c + 2);
            *(float4*)(row + c) = make_float4(a.x, a.y, b.x, b.y);
            ss += (a.x * a.x + a.y * a.y) + (b.x * b.x + b.y * b.y);
        }
    } else {
#pragma unroll 4
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float d = delta.load(base + c);
            row[c] = d;
            ss += d * d;
        }
    }
    ss = block_sum(ss, scratch);
    const float rd = rsqrtf(ss / (float)hidden + eps_d);
    float sx = 0.f;
    if (quad) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float4 xv = *(const float4*)(x + base + c), dv = *(const float4*)(row + c), wv = *(const float4*)(wd + c);
            const float4 v = make_float4(xv.x + dv.x * rd * wv.x, xv.y + dv.y * rd * wv.y, xv.z + dv.z * rd * wv.z,
                                         xv.w + dv.w * rd * wv.w);
            *(float4*)(x + base + c) = v;
            *(float4*)(row + c) = v;
            sx += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            if (raw != nullptr) { st2(raw + base + c, v.x, v.y); st2(raw + base + c + 2, v.z, v.w); }
        }
    } else {
#pragma unroll 4
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = x[base + c] + row[c] * rd * wd[c];
            x[base + c] = v;
            row[c] = v;
            sx += v * v;
            if (raw != nullptr) raw[base + c] = from_f32<T>(v);
        }
    }
    if (out == nullptr) return;
    sx = block_sum(sx, scratch);
    const float ro = rsqrtf(sx / (float)hidden + eps_o);
    if (quad) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float4 v = *(const float4*)(row + c), wv = *(const float4*)(wo + c);
            st2(out + base + c, v.x * ro * wv.x, v.y * ro * wv.y);
            st2(out + base + c + 2, v.z * ro * wv.z, v.w * ro * wv.w);
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[base + c] = from_f32<T>(row[c] * ro * wo[c]);
    }
}

// ------------------------------------------------------ gate of the per-layer token input
// g[t][c] = gelu_tanh(z[t][c]) * side[tok[t]][offset + c]
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
template <typename T>
__global__ void __launch_bounds__(128)
token_gate_kernel(GemmOut<T> z, const int* __restrict__ tokens, const T* __restrict__ side, int side_cols,
                  int offset, int dim, T* __restrict__ out, int vocab, const int* __restrict__ deferred,
                  int n_deferred, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = resolve_token(tokens[t], vocab, deferred, n_deferred, err);
    const T* e = side + (long long)tok * side_cols + offset;
    for (int c = threadIdx.x; c < dim; c += blockDim.x)
        out[(long long)t * dim + c] = from_f32<T>(gelu_tanh_f(z.load((long long)t * dim + c)) * to_f32(e[c]));
}

// ------------------------------------------------------ activations of feed-forwards
// out[t][c] = act(up[t][c]) * (c < routed_cols ? route[t][c / per_expert] : 1)
// kind 0: relu(z)^2;  1: z/2 (1 + erf(z / sqrt 2));  2: the tanh form of gelu
template <typename T>
__global__ void __launch_bounds__(256)
ffn_activation_kernel(GemmOut<T> up, T* __restrict__ out, long long n, int cols, int kind,
                      const float* __restrict__ route, int experts, int per_expert, int routed_cols) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float z = up.load(i);
        float a;
        if (kind == 0) {
            const float r = fmaxf(z, 0.f);
            a = r * r;
        } else if (kind == 1) {
            a = 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
        } else {
            a = gelu_tanh_f(z);
        }
        if (route != nullptr) {
            const int c = (int)(i % cols);
            if (c < routed_cols) {
                const float w = route[(i / cols) * experts + c / per_expert];
                a = w == 0.f ? 0.f : a * w;          // an expert that was not chosen adds nothing, whatever it holds
            }
        }
        out[i] = from_f32<T>(a);
    }
}

// The same for bfloat16 rows whose columns come in whole groups of 8: a thread takes 8 neighbouring
// columns of one row (16 bytes in, 16 bytes out); grid (column groups, rows).
__global__ void __launch_bounds__(256)
ffn_activation_vec_kernel(const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ out, int cols, int kind,
                          const float* __restrict__ route, int experts, int per_expert, int routed_cols) {
    pdl_launch_dependents();
    pdl_wait();
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c0 >= cols) return;
    const long long row = blockIdx.y;
    const uint4 raw = *(const uint4*)(up + row * cols + c0);
    const __nv_bfloat162* in2 = (const __nv_bfloat162*)&raw;
    float w = 1.f;
    if (route != nullptr && c0 < routed_cols) w = route[row * experts + c0 / per_expert];
    uint4 res;
    __nv_bfloat162* out2 = (__nv_bfloat162*)&res;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 z = __bfloat1622float2(in2[i]);
        float a[2] = {z.x, z.y};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float v = a[k];
            if (kind == 0) {
                const float r = fmaxf(v, 0.f);
                a[k] = r * r;
            } else if (kind == 1) {
                a[k] = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
            } else {
                a[k] = gelu_tanh_f(v);
            }
            a[k] = w == 0.f ? 0.f : a[k] * w;
        }
        out2[i] = __floats2bfloat162_rn(a[0], a[1]);
    }
    *(uint4*)(out + row * cols + c0) = res;
}

// ------------------------------------------------------ router
// One warp per token: the `top` largest of the token's `experts` float logits (ties to the lower
// index), their softmax, written as a dense row of weights [experts] (zero for the others) and as
// lists idx / wt [top] (largest first).
__global__ void __launch_bounds__(128)
route_topk_kernel(const float* __restrict__ logits, float* __restrict__ route, int* __restrict__ idx,
                  float* __restrict__ wt, int n, int experts, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n) return;
    const float* z = logits + (long long)t * experts;
    float* r = route + (long long)t * experts;
    for (int e = lane; e < experts; e += 32) r[e] = 0.f;
    __syncwarp();
    float zmax = 0.f, sum = 0.f;
    for (int j = 0; j < top; ++j) {
        // the best expert not yet taken (taken ones carry a weight > 0)
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            if (r[e] != 0.f) continue;
            const float v = z[e];
            if (bi == 0x7fffffff || v > best) { best = v; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) break;                 // fewer experts than `top`
        if (j == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == 0) {
            r[bi] = p > 0.f ? p : 1e-30f;             // marks the expert as taken
            idx[(long long)t * top + j] = bi;
            wt[(long long)t * top + j] = p;
        }
        __syncwarp();
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    for (int e = lane; e < experts; e += 32) r[e] *= inv;
    for (int j = lane; j < top; j += 32) wt[(long long)t * top + j] *= inv;
}

}  // namespace

CRANE_API int crane_embed_sinusoid(int dtype, const int* tokens, const int* positions, const void* table,
                                   const double* freq, float* x, float* keep, int n_tokens, int hidden,
                                   int vocab, const int* deferred, int n_deferred, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    DISPATCH_T(dtype, return crane_launch(embed_sinusoid_kernel<T>, dim3(n_tokens), dim3(256), 0, st, tokens,
                                          positions, (const T*)table, freq, x, keep, hidden, vocab, deferred,
                                          n_deferred, err));
}

CRANE_API int crane_stream_enter(float* x, const float* kept, const float* vec, int n_rows, int hidden,
                                 cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const long long n = (long long)n_rows * hidden;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    return crane_launch(stream_enter_kernel, dim3(blocks), dim3(256), 0, st, x, kept, vec, n, hidden);
}

CRANE_API int crane_add_normed_norm(int dtype, float* x, const void* delta, const float* delta_parts,
                                    int n_parts, long long part_stride, const float* wd, const float* wo,
                                    void* out, void* raw, int n_rows, int hidden, float eps_d, float eps_o,
                                    cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    DISPATCH_T(dtype, {
        GemmOut<T> d{(const T*)delta, delta_parts, n_parts, part_stride};
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_normed_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // few rows (a step of single tokens): more threads a row, so that a thread's loads, each of which
        // waits for memory, are few
        const int threads = n_rows <= 64 ? (hidden >= 4096 ? 1024 : hidden >= 1024 ? 512 : 256) : 256;
        return crane_launch(add_normed_norm_kernel<T>, dim3(n_rows), dim3(threads), smem, st, x, d, wd, wo, (T*)out,
                            (T*)raw, hidden, eps_d, eps_o);
    });
}

CRANE_API int crane_token_gate(int dtype, const void* z, const float* z_parts, int n_parts, long long part_stride,
                               const int* tokens, const void* side, int side_cols, int offset, int dim,
                               void* out, int n_tokens, int vocab, const int* deferred, int n_deferred,
                               int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    DISPATCH_T(dtype, {
        GemmOut<T> g{(const T*)z, z_parts, n_parts, part_stride};
        return crane_launch(token_gate_kernel<T>, dim3(n_tokens), dim3(128), 0, st, g, tokens, (const T*)side,
                            side_cols, offset, dim, (T*)out, vocab, deferred, n_deferred, err);
    });
}

CRANE_API int crane_ffn_activation(int dtype, const void* up, const float* up_parts, int n_parts,
                                   long long part_stride, void* out, int n_rows, int cols, int kind,
                                   const float* route, int experts, int per_expert, int routed_cols,
                                   cudaStream_t st) {
    if (n_rows <= 0 || cols <= 0) return 0;
    const long long n = (long long)n_rows * cols;
    const int blocks = (int)((n + 1023) / 1024 < 8192 ? (n + 1023) / 1024 : 8192);
    if (dtype == 1 && up != nullptr && cols % 8 == 0 && n_rows <= 65535 && ((uintptr_t)up | (uintptr_t)out) % 16 == 0 &&
        (route == nullptr || (per_expert % 8 == 0 && routed_cols % 8 == 0)))
        return crane_launch(ffn_activation_vec_kernel, dim3((cols / 8 + 255) / 256, n_rows), dim3(256), 0, st,
                            (const __nv_bfloat16*)up, (__nv_bfloat16*)out, cols, kind, route, experts, per_expert,
                            routed_cols);
    DISPATCH_T(dtype, {
        GemmOut<T> u{(const T*)up, up_parts, n_parts, part_stride};
        return crane_launch(ffn_activation_kernel<T>, dim3(blocks), dim3(256), 0, st, u, (T*)out, n, cols, kind,
                            route, experts, per_expert, routed_cols);
    });
}

CRANE_API int crane_route_topk(const float* logits, float* route, int* idx, float* wt, int n, int experts,
                               int top, cudaStream_t st) {
    if (n <= 0) return 0;
    if (experts <= 0 || top <= 0) return (int)cudaErrorInvalidValue;
    return crane_launch(route_topk_kernel, dim3((n + 3) / 4), dim3(128), 0, st, logits, route, idx, wt, n,
                        experts, top);
}
