// Latent attention, the part around the attention itself: what a token leaves in the cache and what its queries
// become.
//
// A token's down-projections arrive as one float row [q_rank | kv_rank | rot_dim] (one product, float accumulators
// unrounded).  latent_prepare RMS-norms the first q_rank elements with a weight (the query latent, handed on in T for
// the up-projection), RMS-norms the next kv_rank with a weight (the latent c, which is all that keys and values are made
// of) and rotates the last rot_dim by the token's position (the one rotated key part that every head shares), and
// writes c | rotated part as the token's row of its cache page [page_size, kv_rank + rot_dim].  Norms, angles and the
// rotation are float; one rounding to T at the store.
//
// The rotation pairs element i with element i + rot/2 over the first `rot` elements of the part (the rest pass):
// (u, v) -> (u cos - v sin, v cos + u sin), cos and sin [n, rot/2] float for the step's positions.
//
// latent_rotate_q rotates the rotated part of every head's query, q [n, heads, dim + rot_dim], into the last rot_dim
// columns of the attention's query rows [n, heads, kv_rank + rot_dim]; the first kv_rank columns are the head's
// unrotated query carried through the key up-projection (a batched matrix product of the caller), so that a score is
// one dot product with a cached row and a head's output is a weighted sum of cached latents.
#include "common.cuh"

using namespace vapi;

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ down, long long down_stride, const float* __restrict__ wq,
                      const float* __restrict__ wkv, float eps, const float* __restrict__ cosr,
                      const float* __restrict__ sinr, int rot, T* __restrict__ cq, T* __restrict__ cache,
                      const int* __restrict__ slot_mapping, int n, int q_rank, int kv_rank, int rot_dim, int page_size,
                      int num_pages, int* __restrict__ status) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    pdl_trigger();
    const int slot = (cache && t < n) ? slot_mapping[t] : 0;
    pdl_wait();
    if (t >= n) return;
    const float* row = down + (size_t)t * down_stride;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss += row[i] * row[i];
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f32<T>(row[i] * inv * wq[i]);
    }
    if (!cache) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (slot < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    const float* c = row + q_rank;
    float ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss += c[i] * c[i];
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)kv_rank + eps);
    const int width = kv_rank + rot_dim;
    T* dst = cache + ((size_t)page * page_size + off) * width;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_f32<T>(c[i] * inv * wkv[i]);
    const float* kr = c + kv_rank;
    const int half = rot >> 1;
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float v = kr[i];
        if (i < rot) {
            const bool first = i < half;
            const int j = first ? i : i - half;
            const float pv = kr[first ? i + half : i - half];
            const float cs = cosr[(size_t)t * half + j], sn = sinr[(size_t)t * half + j];
            v = first ? v * cs - pv * sn : v * cs + pv * sn;
        }
        dst[kv_rank + i] = from_f32<T>(v);
    }
}

// one warp per (token, head)
template <typename T>
__global__ void latent_rotate_q_kernel(const T* __restrict__ q, long long q_stride, const float* __restrict__ cosr,
                                       const float* __restrict__ sinr, int rot, T* __restrict__ qfull, int n, int heads,
                                       int dim, int rot_dim, int kv_rank) {
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    if (item >= (long long)n * heads) return;
    const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
    const T* src = q + (size_t)t * q_stride + (size_t)h * (dim + rot_dim) + dim;
    T* dst = qfull + ((size_t)t * heads + h) * (kv_rank + rot_dim) + kv_rank;
    const int half = rot >> 1;
    for (int i = lane; i < rot_dim; i += 32) {
        float v = to_f32(src[i]);
        if (i < rot) {
            const bool first = i < half;
            const int j = first ? i : i - half;
            const float pv = to_f32(src[first ? i + half : i - half]);
            const float cs = cosr[(size_t)t * half + j], sn = sinr[(size_t)t * half + j];
            v = first ? v * cs - pv * sn : v * cs + pv * sn;
        }
        dst[i] = from_f32<T>(v);
    }
}

VAPI_EXPORT int vapi_latent_prepare(const float* down, long long down_stride, const float* wq, const float* wkv, float eps,
                                    const float* cosr, const float* sinr, int rot, void* cq, void* cache, int dtype,
                                    const int* slot_mapping, int n, int q_rank, int kv_rank, int rot_dim, int page_size,
                                    int num_pages, int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || down_stride < (long long)q_rank + kv_rank + rot_dim)
        return fail(-1, "latent_prepare: a row of %lld elements for %d + %d + %d", down_stride, q_rank, kv_rank, rot_dim);
    if (rot < 0 || rot > rot_dim || (rot & 1) || (rot > 0 && (!cosr || !sinr)))
        return fail(-1, "latent_prepare: %d rotated elements of %d", rot, rot_dim);
    if (q_rank > 0 && (!wq || !cq)) return fail(-1, "latent_prepare: the query latent needs its weight and its output");
    if (cache && (page_size <= 0 || num_pages <= 0 || !slot_mapping || !wkv))
        return fail(-1, "latent_prepare: cache given without pages, slot mapping or weight");
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(latent_prepare_kernel<float>, n, 128, 0, stream, down, down_stride, wq, wkv, eps, cosr, sinr, rot, (float*)cq,
                   (float*)cache, slot_mapping, n, q_rank, kv_rank, rot_dim, page_size, num_pages, status);
    else if (dtype == VAPI_BF16)
        e = launch(latent_prepare_kernel<__nv_bfloat16>, n, 128, 0, stream, down, down_stride, wq, wkv, eps, cosr, sinr, rot,
                   (__nv_bfloat16*)cq, (__nv_bfloat16*)cache, slot_mapping, n, q_rank, kv_rank, rot_dim, page_size, num_pages,
                   status);
    else
        return fail(-2, "latent_prepare: unsupported dtype %d", dtype);
    return check_launch("latent_prepare", e);
}

VAPI_EXPORT int vapi_latent_rotate_q(const void* q, long long q_stride, const float* cosr, const float* sinr, int rot,
                                     void* qfull, int dtype, int n, int heads, int dim, int rot_dim, int kv_rank,
                                     cudaStream_t stream) {
    if (n <= 0 || rot_dim <= 0) return 0;
    if (heads <= 0 || dim < 0 || kv_rank <= 0 || q_stride < (long long)heads * (dim + rot_dim))
        return fail(-1, "latent_rotate_q: %d heads of %d + %d in rows of %lld", heads, dim, rot_dim, q_stride);
    if (rot < 0 || rot > rot_dim || (rot & 1) || (rot > 0 && (!cosr || !sinr)))
        return fail(-1, "latent_rotate_q: %d rotated elements of %d", rot, rot_dim);
    const long long items = (long long)n * heads;
    const int blocks = (int)((items + 3) / 4);
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(latent_rotate_q_kernel<float>, blocks, 128, 0, stream, (const float*)q, q_stride, cosr, sinr, rot, (float*)qfull,
                   n, heads, dim, rot_dim, kv_rank);
    else if (dtype == VAPI_BF16)
        e = launch(latent_rotate_q_kernel<__nv_bfloat16>, blocks, 128, 0, stream, (const __nv_bfloat16*)q, q_stride, cosr, sinr,
                   rot, (__nv_bfloat16*)qfull, n, heads, dim, rot_dim, kv_rank);
    else
        return fail(-2, "latent_rotate_q: unsupported dtype %d", dtype);
    return check_launch("latent_rotate_q", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
