// Several residual streams side by side (hyper-connections), the layer norm that reads them, and the
// small elementwise steps of mixers that run side by side.
//
// The residual state of a token is S copies of a row, x[t, s, :] (float).  A sublayer reads
// u = sum_s read[s] x_s through a norm, and writes its output y back as
//     x_t <- sum_s mix[s, t] x_s + write[t] y          (all copies at once, from the old ones).
// As with a single stream, a sublayer's output is not written by a pass of its own: it is handed on,
// and the kernel that reads the streams for the next sublayer first applies the pending write, then
// forms u and norms it, one block a token.  S = 1 with mix = write = read = 1 is the ordinary
// residual sum, so the same kernel serves a model with one stream.
//
// Norms: kind 0 is a layer norm with a weight and no bias, (u - mean) / sqrt(var + eps) * w with the
// variance taken as the mean of the squared deviations (two passes over the row, which is kept in
// shared memory); kind 1 is an RMS norm, u / sqrt(mean u^2 + eps) * w.  Sums are float.
#include "common.cuh"

using namespace vapi;

constexpr int HC_MAX_STREAMS = 8;

// x[t, s, c] = table[token[t], c] + (c even ? sin : cos)(position[t] * freq[c / 2]) for every copy s.
// freq is float, rounded once from the exact value; the angle is one float product.
template <typename T>
__global__ void embed_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                      const int* __restrict__ positions, const float* __restrict__ freq,
                                      const T* __restrict__ pos_table, int pos_rows,
                                      float* __restrict__ x, int n, int hidden, int vocab, int streams,
                                      int* __restrict__ status) {
    const int t = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (t >= n) return;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0 && status) atomicExch(status, 1);
        tok = 0;
    }
    const float p = (float)positions[t];
    const T* row = table + (size_t)tok * hidden;
    // a learned position vector: row `position` of a second table, added as it is
    const T* prow = nullptr;
    if (pos_table) {
        int pi = positions[t];
        if (pi < 0 || pi >= pos_rows) {
            if (threadIdx.x == 0 && status) atomicExch(status, 5);
            pi = 0;
        }
        prow = pos_table + (size_t)pi * hidden;
    }
    float* xr = x + (size_t)t * streams * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = to_f32(row[c]);
        if (freq) {
            const float angle = p * freq[c >> 1];
            v += (c & 1) ? cosf(angle) : sinf(angle);
        }
        if (prow) v += to_f32(prow[c]);
        for (int s = 0; s < streams; ++s) xr[(size_t)s * hidden + c] = v;
    }
}

VAPI_EXPORT int vapi_embed_sinusoid(const void* table, int dtype, const int* tokens, const int* positions,
                                    const float* freq, const void* pos_table, int pos_rows, float* x, int n, int hidden,
                                    int vocab, int streams, int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || streams < 1 || streams > HC_MAX_STREAMS)
        return fail(-1, "embed_sinusoid: hidden=%d vocab=%d streams=%d", hidden, vocab, streams);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(embed_sinusoid_kernel<float>, n, threads, 0, stream, (const float*)table, tokens, positions, freq,
                   (const float*)pos_table, pos_rows, x, n, hidden, vocab, streams, status);
    else if (dtype == VAPI_BF16)
        e = launch(embed_sinusoid_kernel<__nv_bfloat16>, n, threads, 0, stream, (const __nv_bfloat16*)table, tokens, positions,
                   freq, (const __nv_bfloat16*)pos_table, pos_rows, x, n, hidden, vocab, streams, status);
    else
        return fail(-2, "embed_sinusoid: unsupported dtype %d", dtype);
    return check_launch("embed_sinusoid", e);
}

// What is pending may also be two mixers' outputs that still want their own RMS norms and their mean:
// y = y_scale * (rms(y) * wy + rms(y2) * wy2)  (wy null: y as it is; y2 null: one branch).
struct HyperArgs {
    const float* mix; const float* write; const float* read;      // [S, S] indexed [from, to]; [S]; [S] (null: ones)
    const float* w; float eps; int kind;                          // the reader's norm (w null: only update the streams)
    const float* wy; const float* wy2; float eps_y; float y_scale;
    const int* rows; int n_out, hidden, streams, write_x;
};

template <typename T> struct Ld4T;
template <> struct Ld4T<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Ld4T<__nv_bfloat16> {
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

// One block a wanted row, any sizes.  y (may be null: nothing pending), mix [S, S] indexed [from, to], write [S],
// read [S] (null: every copy counts once).  With `rows` the streams are left as they are (the pending
// write is applied on the fly).  w null: only the streams are updated.
template <typename T>
__global__ void hyper_read_norm_kernel(float* __restrict__ x, const T* __restrict__ y, const T* __restrict__ y2, HyperArgs p,
                                       T* __restrict__ out) {
    extern __shared__ float hc_row[];          // the row u, [hidden]
    __shared__ float red[33];
    __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_write[HC_MAX_STREAMS], s_read[HC_MAX_STREAMS];
    const int j = blockIdx.x;
    const int streams = p.streams, hidden = p.hidden;
    pdl_trigger();
    if (threadIdx.x < streams * streams) s_mix[threadIdx.x] = (y && p.mix) ? p.mix[threadIdx.x] : 0.f;
    if (threadIdx.x < streams) {
        s_write[threadIdx.x] = (y && p.write) ? p.write[threadIdx.x] : 0.f;
        s_read[threadIdx.x] = p.read ? p.read[threadIdx.x] : 1.f;
    }
    pdl_wait();
    if (j >= p.n_out) return;
    __syncthreads();
    const int row = p.rows ? p.rows[j] : j;
    float* xr = x + (size_t)row * streams * hidden;
    const T* yr = y ? y + (size_t)row * hidden : nullptr;
    const T* yr2 = y2 ? y2 + (size_t)row * hidden : nullptr;
    float inv1 = 1.f, inv2 = 0.f;
    if (yr && p.wy) {
        float s1 = 0.f, s2 = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float a = to_f32(yr[c]), b = yr2 ? to_f32(yr2[c]) : 0.f;
            s1 += a * a;
            s2 += b * b;
        }
        s1 = block_sum(s1, red);
        s2 = block_sum(s2, red);
        inv1 = rsqrtf(s1 / (float)hidden + p.eps_y);
        inv2 = rsqrtf(s2 / (float)hidden + p.eps_y);
    }
    float sum = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float old[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) old[s] = s < streams ? xr[(size_t)s * hidden + c] : 0.f;
        float u = 0.f;
        if (yr) {
            float yv = to_f32(yr[c]);
            if (p.wy) {
                yv = yv * inv1 * p.wy[c];
                if (yr2) yv += to_f32(yr2[c]) * inv2 * p.wy2[c];
                yv = round_to<T>(yv * p.y_scale);       // what a kernel of its own would have stored
            }
#pragma unroll
            for (int t = 0; t < HC_MAX_STREAMS; ++t) {
                if (t < streams) {
                    float v = s_write[t] * yv;
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; ++s)
                        if (s < streams) v = fmaf(s_mix[s * streams + t], old[s], v);
                    if (p.write_x) xr[(size_t)t * hidden + c] = v;
                    u = fmaf(s_read[t], v, u);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < HC_MAX_STREAMS; ++t)
                if (t < streams) u = fmaf(s_read[t], old[t], u);
        }
        hc_row[c] = u;
        sum += p.kind == 0 ? u : u * u;
    }
    if (!p.w) return;
    sum = block_sum(sum, red);
    float mean = 0.f, inv;
    if (p.kind == 0) {
        mean = sum / (float)hidden;
        float dev = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float d = hc_row[c] - mean;      // each thread reads back what it wrote itself
            dev += d * d;
        }
        dev = block_sum(dev, red);
        inv = rsqrtf(dev / (float)hidden + p.eps);
    } else {
        inv = rsqrtf(sum / (float)hidden + p.eps);
    }
    T* orow = out + (size_t)j * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) orow[c] = from_f32<T>((hc_row[c] - mean) * inv * p.w[c]);
}

// The same with 16-byte accesses and the row u held in registers between the passes, for S streams known at
// compile time and hidden a multiple of 4, at most 4 * HC_KMAX * blockDim.
constexpr int HC_KMAX = 4;
template <typename T, int S>
__global__ void hyper_read_norm_vec_kernel(float* __restrict__ x, const T* __restrict__ y, const T* __restrict__ y2, HyperArgs p,
                                           T* __restrict__ out) {
    __shared__ float red[33];
    __shared__ float s_mix[S * S], s_write[S], s_read[S];
    const int j = blockIdx.x;
    const int hidden = p.hidden, h4 = hidden >> 2;
    pdl_trigger();
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = (y && p.mix) ? p.mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_write[threadIdx.x] = (y && p.write) ? p.write[threadIdx.x] : 0.f;
        s_read[threadIdx.x] = p.read ? p.read[threadIdx.x] : 1.f;
    }
    pdl_wait();
    if (j >= p.n_out) return;
    __syncthreads();
    const int row = p.rows ? p.rows[j] : j;
    float* xr = x + (size_t)row * S * hidden;
    const T* yr = y ? y + (size_t)row * hidden : nullptr;
    const T* yr2 = y2 ? y2 + (size_t)row * hidden : nullptr;
    float inv1 = 1.f, inv2 = 0.f;
    if (yr && p.wy) {
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < HC_KMAX; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < h4) {
                const float4 a = Ld4T<T>::load(yr + 4 * c);
                s1 += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                if (yr2) {
                    const float4 b = Ld4T<T>::load(yr2 + 4 * c);
                    s2 += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
                }
            }
        }
        s1 = block_sum(s1, red);
        s2 = block_sum(s2, red);
        inv1 = rsqrtf(s1 / (float)hidden + p.eps_y);
        inv2 = rsqrtf(s2 / (float)hidden + p.eps_y);
    }
    float4 u4[HC_KMAX];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < HC_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        u4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c >= h4) continue;
        float old[S][4];
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const float4 v = Ld4T<float>::load(xr + (size_t)s * hidden + 4 * c);
            old[s][0] = v.x; old[s][1] = v.y; old[s][2] = v.z; old[s][3] = v.w;
        }
        float uu[4] = {0.f, 0.f, 0.f, 0.f};
        if (yr) {
            const float4 ya = Ld4T<T>::load(yr + 4 * c);
            float yv[4] = {ya.x, ya.y, ya.z, ya.w};
            if (p.wy) {
                const float4 wa = Ld4T<float>::load(p.wy + 4 * c);
                const float wv[4] = {wa.x, wa.y, wa.z, wa.w};
                float bv[4] = {0.f, 0.f, 0.f, 0.f}, w2[4] = {0.f, 0.f, 0.f, 0.f};
                if (yr2) {
                    const float4 yb = Ld4T<T>::load(yr2 + 4 * c), wb = Ld4T<float>::load(p.wy2 + 4 * c);
                    bv[0] = yb.x; bv[1] = yb.y; bv[2] = yb.z; bv[3] = yb.w;
                    w2[0] = wb.x; w2[1] = wb.y; w2[2] = wb.z; w2[3] = wb.w;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = yv[e] * inv1 * wv[e];
                    if (yr2) v += bv[e] * inv2 * w2[e];
                    yv[e] = round_to<T>(v * p.y_scale);
                }
            }
#pragma unroll
            for (int t = 0; t < S; ++t) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[e] = s_write[t] * yv[e];
#pragma unroll
                    for (int s = 0; s < S; ++s) v[e] = fmaf(s_mix[s * S + t], old[s][e], v[e]);
                    uu[e] = fmaf(s_read[t], v[e], uu[e]);
                }
                if (p.write_x) Ld4T<float>::store(xr + (size_t)t * hidden + 4 * c, make_float4(v[0], v[1], v[2], v[3]));
            }
        } else {
#pragma unroll
            for (int t = 0; t < S; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) uu[e] = fmaf(s_read[t], old[t][e], uu[e]);
        }
        u4[k] = make_float4(uu[0], uu[1], uu[2], uu[3]);
        sum += p.kind == 0 ? (uu[0] + uu[1]) + (uu[2] + uu[3]) : uu[0] * uu[0] + uu[1] * uu[1] + uu[2] * uu[2] + uu[3] * uu[3];
    }
    if (!p.w) return;
    sum = block_sum(sum, red);
    float mean = 0.f, inv;
    if (p.kind == 0) {
        mean = sum / (float)hidden;
        float dev = 0.f;
#pragma unroll
        for (int k = 0; k < HC_KMAX; ++k) {
            if ((int)(threadIdx.x + k * blockDim.x) < h4) {
                const float a = u4[k].x - mean, b = u4[k].y - mean, c = u4[k].z - mean, d = u4[k].w - mean;
                dev += a * a + b * b + c * c + d * d;
            }
        }
        dev = block_sum(dev, red);
        inv = rsqrtf(dev / (float)hidden + p.eps);
    } else {
        inv = rsqrtf(sum / (float)hidden + p.eps);
    }
    T* orow = out + (size_t)j * hidden;
#pragma unroll
    for (int k = 0; k < HC_KMAX; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < h4) {
            const float4 wv = Ld4T<float>::load(p.w + 4 * c);
            Ld4T<T>::store(orow + 4 * c, make_float4((u4[k].x - mean) * inv * wv.x, (u4[k].y - mean) * inv * wv.y,
                                                     (u4[k].z - mean) * inv * wv.z, (u4[k].w - mean) * inv * wv.w));
        }
    }
}

template <typename T>
static int launch_hyper(float* x, const void* y, const void* y2, const HyperArgs& p, void* out, cudaStream_t stream) {
    const int hidden = p.hidden;
    cudaError_t e;
    const int vt = hidden >= 2048 ? 256 : 128;
    const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)y2 | (uintptr_t)out | (uintptr_t)p.w | (uintptr_t)p.wy |
                           (uintptr_t)p.wy2) & 15) == 0;
    if (hidden % 4 == 0 && hidden / 4 <= HC_KMAX * vt && p.streams <= 4 && aligned) {
#define HC_VEC(S) e = launch(hyper_read_norm_vec_kernel<T, S>, p.n_out, vt, 0, stream, x, (const T*)y, (const T*)y2, p, (T*)out)
        if (p.streams == 1) HC_VEC(1);
        else if (p.streams == 2) HC_VEC(2);
        else if (p.streams == 3) HC_VEC(3);
        else HC_VEC(4);
#undef HC_VEC
        return check_launch("hyper_read_norm", e);
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return fail(-1, "hyper_read_norm: rows of %d do not fit shared memory", hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    auto kern = hyper_read_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch(kern, p.n_out, threads, smem, stream, x, (const T*)y, (const T*)y2, p, (T*)out);
    return check_launch("hyper_read_norm", e);
}

VAPI_EXPORT int vapi_hyper_read_norm(float* x, const void* y, const void* y2, int dtype, const float* wy, const float* wy2,
                                     float eps_y, float y_scale, const float* mix, const float* write, const float* read,
                                     const float* w, float eps, int kind, const int* rows, void* out, int n_out, int hidden,
                                     int streams, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (hidden <= 0 || streams < 1 || streams > HC_MAX_STREAMS)
        return fail(-1, "hyper_read_norm: hidden=%d streams=%d (at most %d)", hidden, streams, HC_MAX_STREAMS);
    if (y && (!mix || !write)) return fail(-1, "hyper_read_norm: a pending output needs its mix matrix and write vector");
    if (y2 && (!y || !wy || !wy2)) return fail(-1, "hyper_read_norm: a second branch needs the first and both norm weights");
    if (w && !out) return fail(-1, "hyper_read_norm: a norm needs an output");
    if (kind != 0 && kind != 1) return fail(-1, "hyper_read_norm: norm kind %d", kind);
    HyperArgs p;
    p.mix = mix; p.write = write; p.read = read; p.w = w; p.eps = eps; p.kind = kind;
    p.wy = wy; p.wy2 = wy2; p.eps_y = eps_y; p.y_scale = y_scale;
    p.rows = rows; p.n_out = n_out; p.hidden = hidden; p.streams = streams; p.write_x = rows ? 0 : 1;
    if (dtype == VAPI_F32) return launch_hyper<float>(x, y, y2, p, out, stream);
    if (dtype == VAPI_BF16) return launch_hyper<__nv_bfloat16>(x, y, y2, p, out, stream);
    return fail(-2, "hyper_read_norm: unsupported dtype %d", dtype);
}

// out[t, :] = scale * sum_b rmsnorm(a_b[t, :]) * w_b  for up to four branches: what mixers that run side by
// side on one input leave.  One block a row; the branch rows are read twice (the second time from cache).
constexpr int BR_MAX = 4;
template <typename T>
struct BranchPtrs {
    const T* a[BR_MAX];
    const float* w[BR_MAX];
};

template <typename T>
__global__ void branch_rmsnorm_mean_kernel(BranchPtrs<T> p, int branches, float eps, float scale, T* __restrict__ out, int n,
                                           int hidden) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (t >= n) return;
    float inv[BR_MAX];
#pragma unroll
    for (int b = 0; b < BR_MAX; ++b) {
        inv[b] = 0.f;
        if (b < branches) {
            const T* r = p.a[b] + (size_t)t * hidden;
            float ss = 0.f;
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
                const float v = to_f32(r[c]);
                ss += v * v;
            }
            ss = block_sum(ss, red);
            inv[b] = rsqrtf(ss / (float)hidden + eps);
        }
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < BR_MAX; ++b)
            if (b < branches) acc += to_f32(p.a[b][(size_t)t * hidden + c]) * inv[b] * p.w[b][c];
        out[(size_t)t * hidden + c] = from_f32<T>(acc * scale);
    }
}

VAPI_EXPORT int vapi_branch_rmsnorm_mean(const void* const* a, const float* const* w, int branches, int dtype, float eps,
                                         float scale, void* out, int n, int hidden, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (branches < 1 || branches > BR_MAX || hidden <= 0)
        return fail(-1, "branch_rmsnorm_mean: %d branches (at most %d), hidden=%d", branches, BR_MAX, hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaError_t e;
    if (dtype == VAPI_F32) {
        BranchPtrs<float> p = {};
        for (int b = 0; b < branches; ++b) { p.a[b] = (const float*)a[b]; p.w[b] = w[b]; }
        e = launch(branch_rmsnorm_mean_kernel<float>, n, threads, 0, stream, p, branches, eps, scale, (float*)out, n, hidden);
    } else if (dtype == VAPI_BF16) {
        BranchPtrs<__nv_bfloat16> p = {};
        for (int b = 0; b < branches; ++b) { p.a[b] = (const __nv_bfloat16*)a[b]; p.w[b] = w[b]; }
        e = launch(branch_rmsnorm_mean_kernel<__nv_bfloat16>, n, threads, 0, stream, p, branches, eps, scale,
                   (__nv_bfloat16*)out, n, hidden);
    } else {
        return fail(-2, "branch_rmsnorm_mean: unsupported dtype %d", dtype);
    }
    return check_launch("branch_rmsnorm_mean", e);
}

// out[t, c] = y[t, c] * sigmoid(g[t * g_stride + c]): a gate as wide as what it multiplies.
template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ y, const T* __restrict__ g, long long g_stride,
                                    T* __restrict__ out, long long total, int width) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= total) return;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const float gv = to_f32(g[(size_t)t * g_stride + c]);
    out[i] = from_f32<T>(to_f32(y[i]) * (1.f / (1.f + expf(-gv))));
}

// 16 bytes a thread (width and the gate's row stride multiples of 8, pointers 16-byte aligned)
__global__ void sigmoid_gate_bf16x8_kernel(const uint4* __restrict__ y, const __nv_bfloat16* __restrict__ g, long long g_stride,
                                           uint4* __restrict__ out, long long total8, int width8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= total8) return;
    const long long t = i / width8;
    const int c8 = (int)(i - t * width8);
    uint4 yv = y[i];
    const uint4 gv = *reinterpret_cast<const uint4*>(g + (size_t)t * g_stride + (size_t)c8 * 8);
    unsigned* yw = reinterpret_cast<unsigned*>(&yv);
    const unsigned* gw = reinterpret_cast<const unsigned*>(&gv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yw[k]));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
        __nv_bfloat162 r = __floats2bfloat162_rn(a.x * (1.f / (1.f + expf(-b.x))), a.y * (1.f / (1.f + expf(-b.y))));
        yw[k] = *reinterpret_cast<unsigned*>(&r);
    }
    out[i] = yv;
}

VAPI_EXPORT int vapi_sigmoid_gate(const void* y, const void* g, long long g_stride, int dtype, void* out, int n, int width,
                                  cudaStream_t stream) {
    if (n <= 0 || width <= 0) return 0;
    if (dtype == VAPI_BF16 && width % 8 == 0 && g_stride % 8 == 0 && (((uintptr_t)y | (uintptr_t)g | (uintptr_t)out) & 15) == 0) {
        const long long total8 = (long long)n * (width / 8);
        return check_launch("sigmoid_gate", launch(sigmoid_gate_bf16x8_kernel, (int)((total8 + 255) / 256), 256, 0, stream,
                                                   (const uint4*)y, (const __nv_bfloat16*)g, g_stride, (uint4*)out, total8, width / 8));
    }
    const long long total = (long long)n * width;
    const int blocks = (int)((total + 255) / 256);
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, (const float*)y, (const float*)g, g_stride, (float*)out,
                   total, width);
    else if (dtype == VAPI_BF16)
        e = launch(sigmoid_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)y, (const __nv_bfloat16*)g,
                   g_stride, (__nv_bfloat16*)out, total, width);
    else
        return fail(-2, "sigmoid_gate: unsupported dtype %d", dtype);
    return check_launch("sigmoid_gate", e);
}

// x <- cap * tanh(x / cap) in place (float logits).
__global__ void softcap_kernel(float* __restrict__ x, float cap, float inv_cap, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i < total) x[i] = cap * tanhf(x[i] * inv_cap);
}

VAPI_EXPORT int vapi_softcap(float* x, float cap, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return fail(-1, "softcap: the cap must be positive");
    return check_launch("softcap", launch(softcap_kernel, (int)((total + 255) / 256), 256, 0, stream, x, cap, 1.f / cap, total));
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
