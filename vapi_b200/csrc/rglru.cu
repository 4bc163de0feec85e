// The real-gated linear recurrent unit: a diagonal linear recurrence whose decay and input gate are
// computed from the token's own input by block-diagonal matrices.
//
// For a token with input u [C] (C channels in `blocks` equal parts of bs; part b has matrices
// Ra[b], Ri[b] of [bs, bs], stored [out, in], and biases):
//     r = sigmoid(Ra[b] u_b + ra_b),   i = sigmoid(Ri[b] u_b + ri_b)
//     log a = -c * r * softplus(lam),  a = exp(log a)
//     S <- a * S + sqrt(1 - a^2) * (i * u),        out = S * gelu_tanh(y)      (y: the other branch)
// The state S [C] is float, one row per request in its slot; a sequence whose portion starts at
// position 0 starts from zeros whatever the slot holds.  Gates, decays and the state are float whatever
// the activation type; u and y arrive in the activation type.
//
// Two kernels.  The first computes, for every token of the step at once, a and g = sqrt(1 - a^2) i u
// (a small float matrix product per part, 64 tokens x 64 channels a block).  The second walks each
// sequence: a block owns 32 channels of one sequence and cuts the portion into as many segments as it
// has warps; every warp first scans its segment from zero (keeping the product of its decays and its
// end value), the segments' carries are chained, and every warp scans its segment again from its
// carry, writing the outputs.  A decode step is the same call with one token a sequence (one warp).
#include "common.cuh"
#include "mma_tile.cuh"

using namespace vapi;

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rg_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// a = exp(log a) for log a <= 0.  What the recurrence feels of a slow decay is 1 - a, so close to one a must be the
// float nearest to the true value: expm1f is exact to an ulp of the small number, and the sum with one rounds once.
// (expf alone may be two ulps of a off, which at a = 0.999 is an error of a part in ten thousand in the decay.)
__device__ __forceinline__ float rg_decay(float log_a) { return log_a > -0.5f ? 1.f + expm1f(log_a) : expf(log_a); }
__device__ __forceinline__ float rg_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

constexpr int RG_TM = 64, RG_TN = 64, RG_TK = 16;
constexpr int RG_UN = 8;                  // tokens whose loads a lane of the scan keeps in flight

template <typename T>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const T* __restrict__ u, long long u_stride, const T* __restrict__ wa, const float* __restrict__ ba,
                   const T* __restrict__ wi, const float* __restrict__ bi, const float* __restrict__ lam, float decay_c,
                   float* __restrict__ a_out, float* __restrict__ g_out, int n, int channels, int bs) {
    __shared__ float Us[RG_TK][RG_TM + 4];
    __shared__ float Was[RG_TK][RG_TN + 4];
    __shared__ float Wis[RG_TK][RG_TN + 4];
    const int b = blockIdx.z;
    const int t0 = blockIdx.x * RG_TM, c0 = blockIdx.y * RG_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* wab = wa + (size_t)b * bs * bs;
    const T* wib = wi + (size_t)b * bs * bs;
    pdl_trigger();
    pdl_wait();
    float acc_a[4][4], acc_i[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc_a[i][j] = acc_i[i][j] = 0.f;
    for (int k0 = 0; k0 < bs; k0 += RG_TK) {
        for (int idx = threadIdx.x; idx < RG_TM * RG_TK; idx += 256) {
            const int tt = idx / RG_TK, kk = idx - tt * RG_TK;
            const int t = t0 + tt, k = k0 + kk;
            Us[kk][tt] = (t < n && k < bs) ? to_f32(u[(size_t)t * u_stride + (size_t)b * bs + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < RG_TN * RG_TK; idx += 256) {
            const int cc = idx / RG_TK, kk = idx - cc * RG_TK;
            const int c = c0 + cc, k = k0 + kk;
            const bool ok = c < bs && k < bs;
            Was[kk][cc] = ok ? to_f32(wab[(size_t)c * bs + k]) : 0.f;
            Wis[kk][cc] = ok ? to_f32(wib[(size_t)c * bs + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RG_TK; ++kk) {
            const float4 uv = *reinterpret_cast<const float4*>(&Us[kk][ty * 4]);
            const float4 av = *reinterpret_cast<const float4*>(&Was[kk][tx * 4]);
            const float4 iv = *reinterpret_cast<const float4*>(&Wis[kk][tx * 4]);
            const float uu[4] = {uv.x, uv.y, uv.z, uv.w};
            const float aa[4] = {av.x, av.y, av.z, av.w};
            const float ii[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc_a[i][j] = fmaf(uu[i], aa[j], acc_a[i][j]);
                    acc_i[i][j] = fmaf(uu[i], ii[j], acc_i[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cb = c0 + tx * 4 + j;
            if (cb >= bs) continue;
            const int c = b * bs + cb;
            const float r = rg_sigmoid(acc_a[i][j] + ba[c]);
            const float ig = rg_sigmoid(acc_i[i][j] + bi[c]);
            const float log_a = -decay_c * r * rg_softplus(lam[c]);
            const float a = rg_decay(log_a);
            const float mult = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));        // sqrt(1 - a^2), exact near a = 1
            const float uv = to_f32(u[(size_t)t * u_stride + c]);
            a_out[(size_t)t * channels + c] = a;
            g_out[(size_t)t * channels + c] = mult * ig * uv;
        }
    }
}

// The gates on the tensor cores, for bfloat16 inputs and matrices (their products are exact in float, and the sums
// are float: nothing is rounded that the float kernel above does not round).  A block takes 64 tokens x 32
// channels of one part: rows 0..31 of its weight tile are the channels' rows of Ra, rows 32..63 those of Ri, so
// the two warps on the left hold r, the two on the right i, and they meet through shared memory.
__global__ void __launch_bounds__(MT_THREADS)
rglru_gates_mma_kernel(const __nv_bfloat16* __restrict__ u, long long u_stride, const __nv_bfloat16* __restrict__ wa,
                       const float* __restrict__ ba, const __nv_bfloat16* __restrict__ wi, const float* __restrict__ bi,
                       const float* __restrict__ lam, float decay_c, float* __restrict__ a_out, float* __restrict__ g_out, int n,
                       int channels, int bs) {
    extern __shared__ __align__(128) unsigned char rg_tile_smem[];
    __shared__ const __nv_bfloat16* a_rows[MT_BM];
    __shared__ const __nv_bfloat16* w_rows[MT_BN];
    const int b = blockIdx.z;
    const int t0 = blockIdx.x * MT_BM, c0 = blockIdx.y * 32;
    pdl_trigger();
    if (threadIdx.x < MT_BM) {
        const int r = threadIdx.x;
        a_rows[r] = t0 + r < n ? u + (size_t)(t0 + r) * u_stride + (size_t)b * bs : nullptr;
        const int c = c0 + (r & 31);
        const __nv_bfloat16* base = (r < 32 ? wa : wi) + (size_t)b * bs * bs;
        w_rows[r] = c < bs ? base + (size_t)c * bs : nullptr;
    }
    pdl_wait();
    __syncthreads();
    float acc[2][4][4];
    mma_tile_64x64(a_rows, w_rows, bs, wa, reinterpret_cast<__nv_bfloat16*>(rg_tile_smem), acc);
    // both gates' sums go through shared memory, so that a warp then owns whole rows of 32 channels: its global
    // reads and writes are whole lines, and a lane's channel (with its bias and decay parameter) never changes
    float* sr = reinterpret_cast<float*>(rg_tile_smem);          // [64][33]: the recurrence gate's sums
    float* si = sr + 64 * 33;                                    // [64][33]: the input gate's sums
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
    float* dst = wn == 0 ? sr : si;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    dst[(wm * 32 + mi * 16 + g + 8 * h) * 33 + ni * 8 + 2 * t + e] = acc[mi][ni][2 * h + e];
    __syncthreads();
    const int cb = c0 + lane;
    if (cb >= bs) return;
    const int c = b * bs + cb;
    const float bias_a = ba[c], bias_i = bi[c], sp = decay_c * rg_softplus(lam[c]);
    for (int row = warp; row < MT_BM; row += MT_THREADS / 32) {
        const int tok = t0 + row;
        if (tok >= n) break;
        const float r = rg_sigmoid(sr[row * 33 + lane] + bias_a);
        const float ig = rg_sigmoid(si[row * 33 + lane] + bias_i);
        const float log_a = -r * sp;
        const float mult = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));
        const float uv = __bfloat162float(u[(size_t)tok * u_stride + c]);
        a_out[(size_t)tok * channels + c] = rg_decay(log_a);
        g_out[(size_t)tok * channels + c] = mult * ig * uv;
    }
}

// grid (sequences, channel groups of 32); block = warps x 32; see the head of the file.
template <typename T>
__global__ void __launch_bounds__(1024)
rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ g, const T* __restrict__ y,
                                  long long y_stride, float* __restrict__ state, long long slot_stride,
                                  const int* __restrict__ state_slots, const int* __restrict__ cu_q,
                                  const int* __restrict__ positions, T* __restrict__ out, int channels, int num_slots,
                                  int* __restrict__ status) {
    extern __shared__ float rg_smem[];         // [warps][2][32]: product of decays, end value
    const int s = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int c = blockIdx.y * 32 + lane;
    pdl_trigger();
    const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0;
    const int slot = state_slots[s];
    pdl_wait();
    if (qlen <= 0) return;
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0 && status) atomicExch(status, 3);
        return;
    }
    const bool ok = c < channels;
    float* st = state + (size_t)slot * slot_stride;
    // read before any warp of the block can have written the new state
    float S = (ok && positions[q0] > 0) ? st[c] : 0.f;
    const int seg = (qlen + warps - 1) / warps;
    const int lo = min(qlen, warp * seg), hi = min(qlen, lo + seg);
    float P = 1.f, E = 0.f;
    if (warps > 1) {
        if (ok) {
            int t = lo;
            for (; t + RG_UN <= hi; t += RG_UN) {          // the loads of several tokens in flight together
                float av[RG_UN], gv[RG_UN];
#pragma unroll
                for (int k = 0; k < RG_UN; ++k) {
                    av[k] = a[(size_t)(q0 + t + k) * channels + c];
                    gv[k] = g[(size_t)(q0 + t + k) * channels + c];
                }
#pragma unroll
                for (int k = 0; k < RG_UN; ++k) {
                    E = fmaf(av[k], E, gv[k]);
                    P *= av[k];
                }
            }
            for (; t < hi; ++t) {
                const float av = a[(size_t)(q0 + t) * channels + c];
                E = fmaf(av, E, g[(size_t)(q0 + t) * channels + c]);
                P *= av;
            }
        }
        rg_smem[(warp * 2) * 32 + lane] = P;
        rg_smem[(warp * 2 + 1) * 32 + lane] = E;
        __syncthreads();
    }
    for (int w = 0; w < warp; ++w) S = fmaf(rg_smem[(w * 2) * 32 + lane], S, rg_smem[(w * 2 + 1) * 32 + lane]);
    if (!ok) return;
    int t = lo;
    for (; t + RG_UN <= hi; t += RG_UN) {
        float av[RG_UN], gv[RG_UN], yv[RG_UN];
#pragma unroll
        for (int k = 0; k < RG_UN; ++k) {
            const size_t row = (size_t)(q0 + t + k);
            av[k] = a[row * channels + c];
            gv[k] = g[row * channels + c];
            yv[k] = to_f32(y[row * y_stride + c]);
        }
#pragma unroll
        for (int k = 0; k < RG_UN; ++k) {
            S = fmaf(av[k], S, gv[k]);
            out[(size_t)(q0 + t + k) * channels + c] = from_f32<T>(S * rg_gelu_tanh(yv[k]));
        }
    }
    for (; t < hi; ++t) {
        const size_t row = (size_t)(q0 + t);
        S = fmaf(a[row * channels + c], S, g[row * channels + c]);
        out[row * channels + c] = from_f32<T>(S * rg_gelu_tanh(to_f32(y[row * y_stride + c])));
    }
    // the warp that owns the portion's last token leaves the state
    if (hi == qlen && lo < hi) st[c] = S;
}

VAPI_EXPORT int vapi_rglru(const void* u, long long u_stride, const void* y, long long y_stride, int dtype, const void* wa,
                           const float* ba, const void* wi, const float* bi, const float* lam, float decay_c,
                           float* a_buf, float* g_buf, float* state, long long slot_stride, const int* state_slots,
                           const int* cu_q, const int* positions, void* out, int n, int num_seqs, int channels, int blocks,
                           int num_slots, int max_q, int* status, cudaStream_t stream) {
    if (n <= 0 || num_seqs <= 0) return 0;
    if (channels <= 0 || blocks <= 0 || channels % blocks) return fail(-1, "rglru: %d channels in %d parts", channels, blocks);
    if (!state || !a_buf || !g_buf) return fail(-1, "rglru: the state and two scratch buffers are needed");
    const int bs = channels / blocks;
    dim3 grid1((n + RG_TM - 1) / RG_TM, (bs + RG_TN - 1) / RG_TN, blocks);
    if (grid1.z > 65535 || grid1.y > 65535) return fail(-1, "rglru: too many parts");
    int warps = (max_q + 31) / 32;
    warps = warps < 1 ? 1 : (warps > 32 ? 32 : warps);
    dim3 grid2(num_seqs, (channels + 31) / 32);
    if (grid2.y > 65535) return fail(-1, "rglru: too many channels");
    const size_t smem = (size_t)warps * 2 * 32 * sizeof(float);
    cudaError_t e;
    if (dtype == VAPI_F32) {
        e = launch(rglru_gates_kernel<float>, grid1, 256, 0, stream, (const float*)u, u_stride, (const float*)wa, ba,
                   (const float*)wi, bi, lam, decay_c, a_buf, g_buf, n, channels, bs);
        int rc = check_launch("rglru_gates", e);
        if (rc != 0) return rc;
        e = launch(rglru_scan_kernel<float>, grid2, warps * 32, smem, stream, (const float*)a_buf, (const float*)g_buf,
                   (const float*)y, y_stride, state, slot_stride, state_slots, cu_q, positions, (float*)out, channels, num_slots,
                   status);
    } else if (dtype == VAPI_BF16) {
        if (bs % 8 == 0 && u_stride % 8 == 0 && ((uintptr_t)u & 15) == 0 && ((uintptr_t)wa & 15) == 0 && ((uintptr_t)wi & 15) == 0) {
            static bool attr_set = false;
            if (!attr_set) {
                if (cudaFuncSetAttribute(rglru_gates_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MT_SMEM) != cudaSuccess)
                    return fail(-101, "rglru: cannot reserve %zu bytes of shared memory", MT_SMEM);
                attr_set = true;
            }
            dim3 grid_tc((n + MT_BM - 1) / MT_BM, (bs + 31) / 32, blocks);
            e = launch(rglru_gates_mma_kernel, grid_tc, MT_THREADS, MT_SMEM, stream, (const __nv_bfloat16*)u, u_stride,
                       (const __nv_bfloat16*)wa, ba, (const __nv_bfloat16*)wi, bi, lam, decay_c, a_buf, g_buf, n, channels, bs);
        } else
        e = launch(rglru_gates_kernel<__nv_bfloat16>, grid1, 256, 0, stream, (const __nv_bfloat16*)u, u_stride,
                   (const __nv_bfloat16*)wa, ba, (const __nv_bfloat16*)wi, bi, lam, decay_c, a_buf, g_buf, n, channels, bs);
        int rc = check_launch("rglru_gates", e);
        if (rc != 0) return rc;
        e = launch(rglru_scan_kernel<__nv_bfloat16>, grid2, warps * 32, smem, stream, (const float*)a_buf, (const float*)g_buf,
                   (const __nv_bfloat16*)y, y_stride, state, slot_stride, state_slots, cu_q, positions, (__nv_bfloat16*)out,
                   channels, num_slots, status);
    } else {
        return fail(-2, "rglru: unsupported dtype %d", dtype);
    }
    return check_launch("rglru_scan", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
