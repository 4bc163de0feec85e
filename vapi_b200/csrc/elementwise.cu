// Embedding gather, fused residual-add + RMSNorm, and SwiGLU.
//
// What the reference does with library calls (candle RmsNorm, residual adds,
// crates/vapi-backend-candle/src/models/lfm2.rs:633-648, 808-817) and one small
// kernel (swiglu, crates/vapi-backend-candle/src/fused.rs:157-165) is done here
// with the residual stream kept in float: the add of a layer's output into the
// stream and the norm that follows are one pass over the row.
#include "common.cuh"

using namespace vapi;

// ---------------------------------------------------------------------------
// embedding: out[r, :] = float(table[tokens[r], :]) * scale
// For a norm that follows (optional): ss = the sum of squares of each produced row, [1][n];
// xw = bfloat16(row * next_w), [n][hidden].
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, float* __restrict__ ss,
                             const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xw,
                             int n, int hidden, int vocab, int* __restrict__ status, float scale) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (r >= n) return;
    int tok = tokens[r];
    if (tok < 0 || tok >= vocab) {  // never read outside the table
        if (threadIdx.x == 0 && status) atomicExch(status, 1);
        tok = 0;
    }
    const TW* src = table + (size_t)tok * hidden;
    float* dst = out + (size_t)r * hidden;
    float acc = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(src[c]) * scale;
        dst[c] = v;
        if (xw) xw[(size_t)r * hidden + c] = __float2bfloat16_rn(v * next_w[c]);
        acc += v * v;
    }
    if (ss) {
        acc = block_sum(acc, red);
        if (threadIdx.x == 0) ss[r] = acc;
    }
}

VAPI_EXPORT int vapi_embed(const void* table, int table_dtype, const int* tokens, float* out,
                           float* ss, const float* next_w, void* xw, int n, int hidden, int vocab,
                           int* status, cudaStream_t stream, float scale) {
    if (xw && !next_w) return fail(-1, "embed: a weighted copy needs the next norm's weight");
    if (n <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return fail(-1, "embed: bad sizes hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dtype == VAPI_F32)
        e = launch(embed_kernel<float>, n, threads, 0, stream, (const float*)table, tokens, out, ss, next_w, (__nv_bfloat16*)xw, n, hidden, vocab, status, scale);
    else if (table_dtype == VAPI_BF16)
        e = launch(embed_kernel<__nv_bfloat16>, n, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, ss, next_w, (__nv_bfloat16*)xw, n, hidden, vocab, status, scale);
    else
        return fail(-2, "embed: unsupported table dtype %d", table_dtype);
    return check_launch("embed", e);
}

// ---------------------------------------------------------------------------
// tokens the host does not know yet: tokens[i] = prev[src[i]] where src[i] >= 0.
// An engine that runs one step ahead enqueues a step before it has read what the step before
// sampled; `prev` is that step's sampled output on the device.  Rows outside `prev` are refused.
__global__ void resolve_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                      const int* __restrict__ prev, int n, int prev_rows,
                                      int* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i < n) {
        const int r = src[i];
        if (r >= 0) {
            if (r < prev_rows) tokens[i] = prev[r];
            else if (status) atomicExch(status, 1);
        }
    }
}

VAPI_EXPORT int vapi_resolve_tokens(int* tokens, const int* src, const int* prev, int n, int prev_rows,
                                    int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!tokens || !src || !prev || prev_rows <= 0) return fail(-1, "resolve_tokens: missing array");
    cudaError_t e = launch(resolve_tokens_kernel, (n + 127) / 128, 128, 0, stream, tokens, src, prev, n, prev_rows, status);
    return check_launch("resolve_tokens", e);
}

// ---------------------------------------------------------------------------
// fused residual add + RMSNorm.
//   if delta: x[row] += float(delta[row])           (x is the float residual stream)
//   out[j]   = T( x[row] * rsqrt(mean(x[row]^2) + eps) * w )
// rows == nullptr: row = j for j in [0, n_out), and x is updated in place.
// rows != nullptr: row = rows[j]; x is NOT written (several j may name one row),
//                  the sum x+delta is formed on the fly.
// Mean and rsqrt in float; the sum of squares is reduced in an order that depends
// only on the block size.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ w, float eps,
                                   const int* __restrict__ rows, T* __restrict__ out,
                                   int n_out, int hidden, int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (dr) {
            v += to_f32(dr[c]);
            if (write_x) xr[c] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    T* orow = out + (size_t)j * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (dr && !write_x) v += to_f32(dr[c]);
        orow[c] = from_f32<T>(v * inv * w[c]);
    }
}

// The same with 16-byte accesses and the row held in registers between the two passes
// (hidden a multiple of 4, at most 4 * 4 * blockDim elements): one read of x and delta, one
// write of x, one write of the output.
template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

constexpr int NORM_KMAX = 4;

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                       const float* __restrict__ w, float eps,
                                       const int* __restrict__ rows, T* __restrict__ out,
                                       int n_out, int hidden, int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
    const int h4 = hidden >> 2;
    float4 v[NORM_KMAX];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < h4) {
            v[k] = Pack4<float>::load(xr + 4 * c);
            if (dr) {
                const float4 d = Pack4<T>::load(dr + 4 * c);
                v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
                if (write_x) Pack4<float>::store(xr + 4 * c, v[k]);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    T* orow = out + (size_t)j * hidden;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            const float4 wv = Pack4<float>::load(w + 4 * c);
            Pack4<T>::store(orow + 4 * c, make_float4(v[k].x * inv * wv.x, v[k].y * inv * wv.y, v[k].z * inv * wv.z, v[k].w * inv * wv.w));
        }
    }
}

VAPI_EXPORT int vapi_add_rmsnorm(float* x, const void* delta, const float* w, float eps,
                                 const int* rows, void* out, int out_dtype, int n_out,
                                 int hidden, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return fail(-1, "add_rmsnorm: hidden=%d", hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int write_x = rows ? 0 : 1;
    cudaError_t e;
    if (hidden % 4 == 0 && hidden <= 4 * NORM_KMAX * 256 && (out_dtype == VAPI_F32 || out_dtype == VAPI_BF16)) {
        const int vt = hidden >= 1024 ? 256 : 128;
        if (hidden / 4 <= NORM_KMAX * vt) {
            if (out_dtype == VAPI_F32)
                e = launch(add_rmsnorm_vec_kernel<float>, n_out, vt, 0, stream, x, (const float*)delta, w, eps, rows, (float*)out, n_out, hidden, write_x);
            else
                e = launch(add_rmsnorm_vec_kernel<__nv_bfloat16>, n_out, vt, 0, stream, x, (const __nv_bfloat16*)delta, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x);
            return check_launch("add_rmsnorm", e);
        }
    }
    if (out_dtype == VAPI_F32)
        e = launch(add_rmsnorm_kernel<float>, n_out, threads, 0, stream, x, (const float*)delta, w, eps, rows, (float*)out, n_out, hidden, write_x);
    else if (out_dtype == VAPI_BF16)
        e = launch(add_rmsnorm_kernel<__nv_bfloat16>, n_out, threads, 0, stream, x, (const __nv_bfloat16*)delta, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x);
    else
        return fail(-2, "add_rmsnorm: unsupported dtype %d", out_dtype);
    return check_launch("add_rmsnorm", e);
}

// Two sublayers side by side, each with a scale per column (layer scale), folded into the stream by the kernel
// that reads it next:  x += s1 * y1 + s2 * y2  (y2 may be absent; a scale may be absent and then counts as one),
// then out = rmsnorm(x) * w, or, without w, the rows of x themselves in T (for a reader that takes the stream as
// it is).  `out` has rows of `out_stride` elements, so that it may be the left part of a wider buffer.  rows as
// for add_rmsnorm.  Everything is float but the two loads and the store.
template <typename T>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ y1, const float* __restrict__ s1,
                                          const T* __restrict__ y2, const float* __restrict__ s2,
                                          const float* __restrict__ w, float eps, const int* __restrict__ rows,
                                          T* __restrict__ out, long long out_stride, int n_out, int hidden, int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* a = y1 ? y1 + (size_t)row * hidden : nullptr;
    const T* b = y2 ? y2 + (size_t)row * hidden : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (a) v += (s1 ? s1[c] : 1.f) * to_f32(a[c]);
        if (b) v += (s2 ? s2[c] : 1.f) * to_f32(b[c]);
        if ((a || b) && write_x) xr[c] = v;
        ss += v * v;
    }
    if (!out) return;
    float inv = 1.f;
    if (w) {
        ss = block_sum(ss, red);
        inv = rsqrtf(ss / (float)hidden + eps);
    }
    T* orow = out + (size_t)j * out_stride;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (!write_x) {
            if (a) v += (s1 ? s1[c] : 1.f) * to_f32(a[c]);
            if (b) v += (s2 ? s2[c] : 1.f) * to_f32(b[c]);
        }
        orow[c] = from_f32<T>(w ? v * inv * w[c] : v);
    }
}

// The same with 16-byte accesses and the row held in registers (hidden a multiple of 4, at most 4 * NORM_KMAX *
// blockDim elements, out_stride a multiple of 4 and every pointer 16-byte aligned).
template <typename T>
__global__ void scaled_add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ y1, const float* __restrict__ s1,
                                              const T* __restrict__ y2, const float* __restrict__ s2,
                                              const float* __restrict__ w, float eps, const int* __restrict__ rows,
                                              T* __restrict__ out, long long out_stride, int n_out, int hidden,
                                              int write_x) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* a = y1 ? y1 + (size_t)row * hidden : nullptr;
    const T* b = y2 ? y2 + (size_t)row * hidden : nullptr;
    const int h4 = hidden >> 2;
    float4 v[NORM_KMAX];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < h4) {
            v[k] = Pack4<float>::load(xr + 4 * c);
            if (a) {
                const float4 d = Pack4<T>::load(a + 4 * c);
                const float4 s = s1 ? Pack4<float>::load(s1 + 4 * c) : make_float4(1.f, 1.f, 1.f, 1.f);
                v[k].x += s.x * d.x; v[k].y += s.y * d.y; v[k].z += s.z * d.z; v[k].w += s.w * d.w;
            }
            if (b) {
                const float4 d = Pack4<T>::load(b + 4 * c);
                const float4 s = s2 ? Pack4<float>::load(s2 + 4 * c) : make_float4(1.f, 1.f, 1.f, 1.f);
                v[k].x += s.x * d.x; v[k].y += s.y * d.y; v[k].z += s.z * d.z; v[k].w += s.w * d.w;
            }
            if ((a || b) && write_x) Pack4<float>::store(xr + 4 * c, v[k]);
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    if (!out) return;
    float inv = 1.f;
    if (w) {
        ss = block_sum(ss, red);
        inv = rsqrtf(ss / (float)hidden + eps);
    }
    T* orow = out + (size_t)j * out_stride;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            float4 o = v[k];
            if (w) {
                const float4 wv = Pack4<float>::load(w + 4 * c);
                o = make_float4(o.x * inv * wv.x, o.y * inv * wv.y, o.z * inv * wv.z, o.w * inv * wv.w);
            }
            Pack4<T>::store(orow + 4 * c, o);
        }
    }
}

VAPI_EXPORT int vapi_scaled_add_rmsnorm(float* x, const void* y1, const float* s1, const void* y2, const float* s2,
                                        const float* w, float eps, const int* rows, void* out, long long out_stride,
                                        int dtype, int n_out, int hidden, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return fail(-1, "scaled_add_rmsnorm: hidden=%d", hidden);
    if (!y1 && y2) return fail(-1, "scaled_add_rmsnorm: the second sublayer comes with a first");
    if (out && out_stride < hidden) return fail(-1, "scaled_add_rmsnorm: output rows of %lld elements for a width of %d", out_stride, hidden);
    if (!out && rows) return fail(-1, "scaled_add_rmsnorm: selected rows leave the stream alone, so an output is needed");
    const int write_x = rows ? 0 : 1;
    const int esz = dtype == VAPI_F32 ? 4 : 2;
    const bool aligned = ((uintptr_t)x & 15) == 0 && (((uintptr_t)y1 | (uintptr_t)y2) & (4 * esz - 1)) == 0 &&
                         (((uintptr_t)s1 | (uintptr_t)s2 | (uintptr_t)w) & 15) == 0 &&
                         ((uintptr_t)out & (4 * esz - 1)) == 0 && out_stride % 4 == 0;
    const int vt = hidden >= 1024 ? 256 : 128;
    const bool vec = hidden % 4 == 0 && hidden / 4 <= NORM_KMAX * vt && aligned;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaError_t e;
#define SAR_GO(T)                                                                                                          \
    e = vec ? launch(scaled_add_rmsnorm_vec_kernel<T>, n_out, vt, 0, stream, x, (const T*)y1, s1, (const T*)y2, s2, w, eps,   \
                     rows, (T*)out, out_stride, n_out, hidden, write_x)                                                       \
            : launch(scaled_add_rmsnorm_kernel<T>, n_out, threads, 0, stream, x, (const T*)y1, s1, (const T*)y2, s2, w, eps,  \
                     rows, (T*)out, out_stride, n_out, hidden, write_x)
    if (dtype == VAPI_F32) SAR_GO(float);
    else if (dtype == VAPI_BF16) SAR_GO(__nv_bfloat16);
    else return fail(-2, "scaled_add_rmsnorm: unsupported dtype %d", dtype);
#undef SAR_GO
    return check_launch("scaled_add_rmsnorm", e);
}

// residual add alone (used at the very end of a step when nothing follows the
// last layer but the stream itself is wanted): x += delta
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) x[i] += to_f32(delta[i]);
}

// x[row] += delta[row]; ss[row] = sum of squares of the new row; xw = bfloat16(new row * next_w)
// (one block per row)
template <typename T>
__global__ void add_residual_ss_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                       float* __restrict__ ss, const float* __restrict__ next_w,
                                       __nv_bfloat16* __restrict__ xw, int n, int hidden) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (r >= n) return;
    float acc = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = x[(size_t)r * hidden + c] + to_f32(delta[(size_t)r * hidden + c]);
        x[(size_t)r * hidden + c] = v;
        if (xw) xw[(size_t)r * hidden + c] = __float2bfloat16_rn(v * next_w[c]);
        acc += v * v;
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) ss[r] = acc;
}

VAPI_EXPORT int vapi_add_residual_ss(float* x, const void* delta, int dtype, float* ss,
                                     const float* next_w, void* xw, int n, int hidden,
                                     cudaStream_t stream) {
    if (n <= 0) return 0;
    if (xw && !next_w) return fail(-1, "add_residual_ss: a weighted copy needs the next norm's weight");
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(add_residual_ss_kernel<float>, n, 256, 0, stream, x, (const float*)delta, ss, next_w, (__nv_bfloat16*)xw, n, hidden);
    else if (dtype == VAPI_BF16)
        e = launch(add_residual_ss_kernel<__nv_bfloat16>, n, 256, 0, stream, x, (const __nv_bfloat16*)delta, ss, next_w, (__nv_bfloat16*)xw, n, hidden);
    else
        return fail(-2, "add_residual_ss: unsupported dtype %d", dtype);
    return check_launch("add_residual_ss", e);
}

VAPI_EXPORT int vapi_add_residual(float* x, const void* delta, int dtype, long long total,
                                  cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(add_residual_kernel<float>, (int)blocks, threads, 0, stream, x, (const float*)delta, (size_t)total);
    else if (dtype == VAPI_BF16)
        e = launch(add_residual_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, x, (const __nv_bfloat16*)delta, (size_t)total);
    else
        return fail(-2, "add_residual: unsupported dtype %d", dtype);
    return check_launch("add_residual", e);
}

// ---------------------------------------------------------------------------
// SwiGLU on a stacked gate/up product: out[r, c] = silu(g[r, c]) * g[r, F + c],
// silu(v) = v / (1 + exp(-v)); float math, one rounding
// (crates/vapi-backend-candle/src/fused.rs:16-25, 157-165).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ g, T* __restrict__ out, int rows, int ff) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rows * ff;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) {
        const size_t r = i / ff, c = i - r * ff;
        const float a = to_f32(g[r * 2 * ff + c]);
        const float b = to_f32(g[r * 2 * ff + ff + c]);
        const float s = a / (1.f + expf(-a));
        out[i] = from_f32<T>(s * b);
    }
}

// four outputs per thread with 16-byte (float) / 8-byte (bfloat16) accesses; ff a multiple of 4
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ g, T* __restrict__ out, int rows, int ff) {
    const int f4 = ff >> 2;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rows * f4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) {
        const size_t r = i / f4, c = (i - r * f4) << 2;
        const float4 a = Pack4<T>::load(g + r * 2 * ff + c);
        const float4 b = Pack4<T>::load(g + r * 2 * ff + ff + c);
        Pack4<T>::store(out + r * ff + c, make_float4(a.x / (1.f + expf(-a.x)) * b.x, a.y / (1.f + expf(-a.y)) * b.y,
                                                      a.z / (1.f + expf(-a.z)) * b.z, a.w / (1.f + expf(-a.w)) * b.w));
    }
}

// bfloat16, ff a multiple of 8: one thread per eight outputs of one row, 16-byte accesses, no
// loop and no index division (the row is the block's y index)
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ out, int ff) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) << 3;
    const size_t r = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    if (c >= ff) return;
    const uint4 a = *reinterpret_cast<const uint4*>(g + r * 2 * ff + c);
    const uint4 b = *reinterpret_cast<const uint4*>(g + r * 2 * ff + ff + c);
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    unsigned o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
        const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
        __nv_bfloat162 y = __floats2bfloat162_rn(x.x / (1.f + expf(-x.x)) * u.x, x.y / (1.f + expf(-x.y)) * u.y);
        o[i] = *reinterpret_cast<unsigned*>(&y);
    }
    *reinterpret_cast<uint4*>(out + r * ff + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

VAPI_EXPORT int vapi_swiglu(const void* g, void* out, int dtype, int rows, int ff,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (ff <= 0) return fail(-1, "swiglu: ff=%d", ff);
    const int threads = 256;
    long long total = (long long)rows * ff;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > sm_count() * 32) blocks = sm_count() * 32;
    cudaError_t e;
    if (dtype == VAPI_BF16 && ff % 8 == 0 && rows <= 65535) {
        const int th = 128;
        dim3 grid((ff / 8 + th - 1) / th, rows);
        e = launch(swiglu_bf16x8_kernel, grid, th, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, ff);
        return check_launch("swiglu", e);
    }
    if (ff % 4 == 0 && (dtype == VAPI_F32 || dtype == VAPI_BF16)) {
        long long vb = (total / 4 + threads - 1) / threads;
        if (vb > sm_count() * 16) vb = sm_count() * 16;
        if (dtype == VAPI_F32) e = launch(swiglu_vec_kernel<float>, (int)vb, threads, 0, stream, (const float*)g, (float*)out, rows, ff);
        else e = launch(swiglu_vec_kernel<__nv_bfloat16>, (int)vb, threads, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, rows, ff);
        return check_launch("swiglu", e);
    }
    if (dtype == VAPI_F32)
        e = launch(swiglu_kernel<float>, (int)blocks, threads, 0, stream, (const float*)g, (float*)out, rows, ff);
    else if (dtype == VAPI_BF16)
        e = launch(swiglu_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, rows, ff);
    else
        return fail(-2, "swiglu: unsupported dtype %d", dtype);
    return check_launch("swiglu", e);
}


// A sublayer's output y, normed on its way into the stream, and the norm that reads the stream
// next, in one pass over the row:
//   x <- x + mult * (y * rsqrt(mean(y^2) + eps_post) * w_post);   out = x * rsqrt(mean(x^2) + eps) * w
// (blocks that norm a sublayer on both sides and scale its contribution).  `y` null: nothing is pending.
// `w` null: no norm follows; with `out` the row itself is handed on in T (a sublayer that reads the stream as
// it is), without it only the stream is updated.  With `rows` the output has one row per entry and x is left
// untouched.
// With `y2` the sublayer was two mixers side by side whose outputs y and y2 are still raw: y stands for
//   scale_b * (y * rsqrt(mean(y^2) + eps_b) * wa + y2 * rsqrt(mean(y2^2) + eps_b) * wb)
// which is formed here, in float, before anything else.
// One block per row; every sum is float.
template <typename T>
__global__ void postnorm_add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ y,
                                            const float* __restrict__ w_post, float eps_post, float mult,
                                            const float* __restrict__ w, float eps,
                                            const int* __restrict__ rows, T* __restrict__ out,
                                            int n_out, int hidden, int write_x, const T* __restrict__ y2,
                                            const float* __restrict__ wa, const float* __restrict__ wb, float eps_b,
                                            float scale_b) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* yr = y ? y + (size_t)row * hidden : nullptr;
    const T* y2r = (y && y2) ? y2 + (size_t)row * hidden : nullptr;
    float inv_a = 0.f, inv_b = 0.f;
    if (y2r) {
        float sa = 0.f, sb = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float a = to_f32(yr[c]), b = to_f32(y2r[c]);
            sa += a * a;
            sb += b * b;
        }
        sa = block_sum(sa, red);
        sb = block_sum(sb, red);
        inv_a = rsqrtf(sa / (float)hidden + eps_b);
        inv_b = rsqrtf(sb / (float)hidden + eps_b);
    }
    auto yval = [&](int c) {
        return y2r ? scale_b * (to_f32(yr[c]) * inv_a * wa[c] + to_f32(y2r[c]) * inv_b * wb[c]) : to_f32(yr[c]);
    };
    float ssy = 0.f;
    for (int c = threadIdx.x; c < hidden && yr; c += blockDim.x) {
        const float v = yval(c);
        ssy += v * v;
    }
    if (yr) ssy = block_sum(ssy, red);
    const float inv_y = rsqrtf(ssy / (float)hidden + eps_post);
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = yr ? xr[c] + mult * (yval(c) * inv_y * w_post[c]) : xr[c];
        if (write_x && yr) xr[c] = v;
        ss += v * v;
    }
    if (!out) return;
    float inv = 1.f;
    if (w) {
        ss = block_sum(ss, red);
        inv = rsqrtf(ss / (float)hidden + eps);
    }
    T* orow = out + (size_t)j * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        // each thread reads back what it wrote itself
        const float v = (write_x || !yr) ? xr[c] : xr[c] + mult * (yval(c) * inv_y * w_post[c]);
        orow[c] = from_f32<T>(w ? v * inv * w[c] : v);
    }
}

// The same with 16-byte accesses and the row held in registers between the passes (hidden a multiple
// of 4, at most 4 * NORM_KMAX * blockDim elements): x, y and the weights are read once, x and the
// output written once.
template <typename T>
__global__ void postnorm_add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ y,
                                                const float* __restrict__ w_post, float eps_post, float mult,
                                                const float* __restrict__ w, float eps,
                                                const int* __restrict__ rows, T* __restrict__ out,
                                                int n_out, int hidden, int write_x, const T* __restrict__ y2,
                                                const float* __restrict__ wa, const float* __restrict__ wb, float eps_b,
                                                float scale_b) {
    __shared__ float red[33];
    const int j = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (j >= n_out) return;
    const int row = rows ? rows[j] : j;
    float* xr = x + (size_t)row * hidden;
    const T* yr = y ? y + (size_t)row * hidden : nullptr;
    const T* y2r = (y && y2) ? y2 + (size_t)row * hidden : nullptr;
    const int h4 = hidden >> 2;
    float4 v[NORM_KMAX];
    float ssy = 0.f;
    if (y2r) {                                   // two raw branches: their norms and their mean come first
        float4 u[NORM_KMAX];
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int k = 0; k < NORM_KMAX; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            v[k] = u[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < h4) {
                v[k] = Pack4<T>::load(yr + 4 * c);
                u[k] = Pack4<T>::load(y2r + 4 * c);
                sa += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
                sb += u[k].x * u[k].x + u[k].y * u[k].y + u[k].z * u[k].z + u[k].w * u[k].w;
            }
        }
        sa = block_sum(sa, red);
        sb = block_sum(sb, red);
        const float inv_a = rsqrtf(sa / (float)hidden + eps_b), inv_b = rsqrtf(sb / (float)hidden + eps_b);
#pragma unroll
        for (int k = 0; k < NORM_KMAX; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < h4) {
                const float4 a4 = Pack4<float>::load(wa + 4 * c), b4 = Pack4<float>::load(wb + 4 * c);
                v[k].x = scale_b * (v[k].x * inv_a * a4.x + u[k].x * inv_b * b4.x);
                v[k].y = scale_b * (v[k].y * inv_a * a4.y + u[k].y * inv_b * b4.y);
                v[k].z = scale_b * (v[k].z * inv_a * a4.z + u[k].z * inv_b * b4.z);
                v[k].w = scale_b * (v[k].w * inv_a * a4.w + u[k].w * inv_b * b4.w);
                ssy += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < NORM_KMAX; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < h4 && yr) {
                v[k] = Pack4<T>::load(yr + 4 * c);
                ssy += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
            }
        }
    }
    if (yr) ssy = block_sum(ssy, red);
    const float inv_y = rsqrtf(ssy / (float)hidden + eps_post);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            const float4 xv = Pack4<float>::load(xr + 4 * c);
            if (yr) {
                const float4 wp = Pack4<float>::load(w_post + 4 * c);
                v[k].x = xv.x + mult * (v[k].x * inv_y * wp.x);
                v[k].y = xv.y + mult * (v[k].y * inv_y * wp.y);
                v[k].z = xv.z + mult * (v[k].z * inv_y * wp.z);
                v[k].w = xv.w + mult * (v[k].w * inv_y * wp.w);
                if (write_x) Pack4<float>::store(xr + 4 * c, v[k]);
            } else {
                v[k] = xv;
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    if (!out) return;
    float inv = 1.f;
    if (w) {
        ss = block_sum(ss, red);
        inv = rsqrtf(ss / (float)hidden + eps);
    }
    T* orow = out + (size_t)j * hidden;
#pragma unroll
    for (int k = 0; k < NORM_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            if (w) {
                const float4 wv = Pack4<float>::load(w + 4 * c);
                Pack4<T>::store(orow + 4 * c, make_float4(v[k].x * inv * wv.x, v[k].y * inv * wv.y, v[k].z * inv * wv.z, v[k].w * inv * wv.w));
            } else {
                Pack4<T>::store(orow + 4 * c, v[k]);
            }
        }
    }
}

VAPI_EXPORT int vapi_postnorm_add_rmsnorm(float* x, const void* y, int dtype, const float* w_post, float eps_post,
                                          float mult, const float* w, float eps, const int* rows, void* out,
                                          int n_out, int hidden, const void* y2, const float* wa, const float* wb,
                                          float eps_b, float scale_b, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0 || (y && !w_post)) return fail(-1, "postnorm_add_rmsnorm: hidden=%d or no weight", hidden);
    if (y2 && (!y || !wa || !wb)) return fail(-1, "postnorm_add_rmsnorm: two branches come with both outputs and both weights");
    if (!y && !out) return 0;
    if (w && !out) return fail(-1, "postnorm_add_rmsnorm: a following norm needs an output");
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int write_x = rows ? 0 : 1;
    cudaError_t e;
    if (hidden % 4 == 0 && (dtype == VAPI_F32 || dtype == VAPI_BF16) && mult != 0.f) {
        const int vt = hidden >= 1024 ? 256 : 128;
        if (hidden / 4 <= NORM_KMAX * vt) {
            if (dtype == VAPI_F32)
                e = launch(postnorm_add_rmsnorm_vec_kernel<float>, n_out, vt, 0, stream, x, (const float*)y, w_post, eps_post,
                           mult, w, eps, rows, (float*)out, n_out, hidden, write_x, (const float*)y2, wa, wb, eps_b, scale_b);
            else
                e = launch(postnorm_add_rmsnorm_vec_kernel<__nv_bfloat16>, n_out, vt, 0, stream, x, (const __nv_bfloat16*)y,
                           w_post, eps_post, mult, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x,
                           (const __nv_bfloat16*)y2, wa, wb, eps_b, scale_b);
            return check_launch("postnorm_add_rmsnorm", e);
        }
    }
    if (dtype == VAPI_F32)
        e = launch(postnorm_add_rmsnorm_kernel<float>, n_out, threads, 0, stream, x, (const float*)y, w_post, eps_post, mult,
                   w, eps, rows, (float*)out, n_out, hidden, write_x, (const float*)y2, wa, wb, eps_b, scale_b);
    else if (dtype == VAPI_BF16)
        e = launch(postnorm_add_rmsnorm_kernel<__nv_bfloat16>, n_out, threads, 0, stream, x, (const __nv_bfloat16*)y, w_post,
                   eps_post, mult, w, eps, rows, (__nv_bfloat16*)out, n_out, hidden, write_x, (const __nv_bfloat16*)y2, wa, wb,
                   eps_b, scale_b);
    else
        return fail(-2, "postnorm_add_rmsnorm: unsupported dtype %d", dtype);
    return check_launch("postnorm_add_rmsnorm", e);
}

// RMS norm over equal groups of a row, with a gate:  out = norm_g(y) * w * silu(z)  (gate_first 0)
// or  out = norm_g(y * silu(z)) * w  (gate_first 1).  y is float [n, width] (what a recurrence
// left), z is T with its own row stride, w has w_len elements and is indexed by column % w_len (one
// weight per head size, or one per column).  `gate_first` carries two bits: bit 0 the order above, bit 1 the
// gate's kind (0: silu(z), 2: sigmoid(z)).  One warp per (row, group).
__device__ __forceinline__ float norm_gate(float zv, int sigmoid_gate) {
    return sigmoid_gate ? 1.f / (1.f + expf(-zv)) : zv / (1.f + expf(-zv));
}

template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                                           const float* __restrict__ w, int w_len, float eps, int gate_first,
                                           T* __restrict__ out, int n, int width, int group) {
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const int groups = width / group;
    const int sig = gate_first & 2;
    gate_first &= 1;
    if (item >= (long long)n * groups) return;
    const int t = (int)(item / groups), g = (int)(item - (long long)t * groups);
    const float* yr = y + (size_t)t * width + (size_t)g * group;
    const T* zr = z + (size_t)t * z_stride + (size_t)g * group;
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) {
        float v = yr[c];
        if (gate_first) {
            const float zv = to_f32(zr[c]);
            v *= norm_gate(zv, sig);
        }
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)group + eps);
    T* orow = out + (size_t)t * width + (size_t)g * group;
    for (int c = lane; c < group; c += 32) {
        const float zv = to_f32(zr[c]);
        const float gate = norm_gate(zv, sig);
        const float wv = w[(g * group + c) % w_len];
        const float v = gate_first ? (yr[c] * gate) * inv * wv : yr[c] * inv * wv * gate;
        orow[c] = from_f32<T>(v);
    }
}

// The same for wide groups (a whole row of a few thousand columns is one group): a block per (row, group).
template <typename T>
__global__ void gated_group_rmsnorm_wide_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                                                const float* __restrict__ w, int w_len, float eps, int gate_first,
                                                T* __restrict__ out, int n, int width, int group) {
    __shared__ float red[33];
    const int groups = width / group;
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups;
    const int sig = gate_first & 2;
    gate_first &= 1;
    pdl_trigger();
    pdl_wait();
    const float* yr = y + (size_t)t * width + (size_t)g * group;
    const T* zr = z + (size_t)t * z_stride + (size_t)g * group;
    float ss = 0.f;
    for (int c = threadIdx.x; c < group; c += blockDim.x) {
        float v = yr[c];
        if (gate_first) {
            const float zv = to_f32(zr[c]);
            v *= norm_gate(zv, sig);
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)group + eps);
    T* orow = out + (size_t)t * width + (size_t)g * group;
    for (int c = threadIdx.x; c < group; c += blockDim.x) {
        const float zv = to_f32(zr[c]);
        const float gate = norm_gate(zv, sig);
        const float wv = w[(g * group + c) % w_len];
        orow[c] = from_f32<T>(gate_first ? (yr[c] * gate) * inv * wv : yr[c] * inv * wv * gate);
    }
}

VAPI_EXPORT int vapi_gated_group_rmsnorm(const float* y, const void* z, long long z_stride, int dtype, const float* w,
                                         int w_len, float eps, int gate_first, void* out, int n, int width, int group,
                                         cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || group <= 0 || width % group || w_len <= 0)
        return fail(-1, "gated_group_rmsnorm: width %d, group %d, weight %d", width, group, w_len);
    const long long items = (long long)n * (width / group);
    const int warps = 4;
    const int blocks = (int)((items + warps - 1) / warps);
    cudaError_t e;
    if (group >= 512 && items <= 0x7fffffffLL && (dtype == VAPI_F32 || dtype == VAPI_BF16)) {
        const int threads = group >= 2048 ? 256 : 128;
        if (dtype == VAPI_F32)
            e = launch(gated_group_rmsnorm_wide_kernel<float>, (int)items, threads, 0, stream, y, (const float*)z, z_stride, w,
                       w_len, eps, gate_first, (float*)out, n, width, group);
        else
            e = launch(gated_group_rmsnorm_wide_kernel<__nv_bfloat16>, (int)items, threads, 0, stream, y, (const __nv_bfloat16*)z,
                       z_stride, w, w_len, eps, gate_first, (__nv_bfloat16*)out, n, width, group);
        return check_launch("gated_group_rmsnorm", e);
    }
    if (dtype == VAPI_F32)
        e = launch(gated_group_rmsnorm_kernel<float>, blocks, warps * 32, 0, stream, y, (const float*)z, z_stride, w, w_len, eps,
                   gate_first, (float*)out, n, width, group);
    else if (dtype == VAPI_BF16)
        e = launch(gated_group_rmsnorm_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, y, (const __nv_bfloat16*)z, z_stride,
                   w, w_len, eps, gate_first, (__nv_bfloat16*)out, n, width, group);
    else
        return fail(-2, "gated_group_rmsnorm: unsupported dtype %d", dtype);
    return check_launch("gated_group_rmsnorm", e);
}

// x *= factor (the output head of a model that scales its logits)
__global__ void scale_kernel(float* __restrict__ x, float factor, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_trigger();
    pdl_wait();
    for (; i < total; i += stride) x[i] *= factor;
}

VAPI_EXPORT int vapi_scale(float* x, float factor, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    long long blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    return check_launch("scale", launch(scale_kernel, (int)blocks, 256, 0, stream, x, factor, (size_t)total));
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
