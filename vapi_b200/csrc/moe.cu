// A mixture of small feed-forward experts: the router, the plan of a step's expert work, the experts'
// two matrix products over tokens grouped by expert, and the weighted sum.
//
// Router (float whatever the activation type): z = Wr h over all `outputs` = experts + identity
// experts; s = softmax(z); the choice score is s + correction; outputs form `groups` equal groups of
// neighbours, a group's score is its largest choice score, and only outputs of the `keep` best groups
// can be chosen (the others count as minus infinity); the `top` largest choice scores win (ties: the
// lower index); their weights are their s divided by the sum of the chosen s (+ 1e-20).  An output
// index >= experts is an identity expert: its output is the input itself.
// A second way of scoring (score_mode 1): the choice is made among the logits z = Wr h + bias themselves, and the
// weights are the softmax over the chosen logits only.
//
// The step's expert work is laid out without the host learning anything about it: after the router, one
// block counts the (token, choice) pairs of each expert in shared memory (a pair's rank within its expert is
// the count it met), turns the counts into offsets, lists the pairs expert by expert and cuts each expert's
// list into tiles of 64 rows.  The two products launch enough blocks for the worst case; a block whose tile does
// not exist returns at once.  up: hid[pos] = relu(W_up[e] h[token])^2, or, for experts with a gate,
// hid[pos] = silu(W_gate[e] h) * (W_up[e] h) from one matrix whose rows alternate gate, up; down: y[pair] = weight *
// W_down[e] hid[pos] in float; the sum over a token's pairs, its identity experts and the shared expert
// is taken in a fixed order.
// The gated form has three constants: out = g' * sigmoid(alpha * g') * (u' + shift) with g' = min(g, limit) and
// u' = clamp(u, -limit, limit) when limit > 0, else g' = g, u' = u.  alpha = 1, shift = 0 and no limit is SiLU gating.
// A third way of choosing needs no router at all (moe_table_route): a table [vocab, top] of expert indices, read at
// the token's id, names the token's experts, each with weight 1 / top.
#include "common.cuh"
#include "mma_tile.cuh"

using namespace vapi;

constexpr int MOE_TM = 64, MOE_TN = 64, MOE_TK = 16;

// Rows of a tile of the experts' products.  The plan and both products of a step must agree on it.  (Tiles of 128 x 128
// on eight warps were measured on prompts of 2,048 tokens over 30 experts: the same time as 64 x 64, because what
// the larger tile gains it loses on the experts' last, partly empty tiles.)
static inline int moe_tile_rows(int pairs, int experts) { (void)pairs; (void)experts; return MOE_TM; }

template <typename T> struct RtLd4;
template <> struct RtLd4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct RtLd4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// One block of four warps per token: the warps share the router's outputs among them (four outputs at a time
// a warp, so that a lane has their loads in flight together), then the first warp chooses.  The order of a
// lane's additions and of a warp's reduction depends on nothing but the width.  shared memory: 2 * outputs
// floats (the scores and the choice scores) + groups floats.
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ corr,
                 const float* __restrict__ bias, int score_mode,
                 int* __restrict__ ids, float* __restrict__ wts, int n, int width, int outputs, int experts, int top,
                 int groups, int keep, int vec4) {
    extern __shared__ float rt_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    float* s = rt_smem;
    float* choice = s + outputs;
    float* gscore = choice + outputs;
    pdl_trigger();
    pdl_wait();
    if (t >= n) return;
    const T* hr = h + (size_t)t * width;
    for (int e0 = warp * 4; e0 < outputs; e0 += warps * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float* w0 = wr + (size_t)e0 * width;
        if (vec4) {
            for (int k = lane * 4; k < width; k += 128) {
                const float4 hv = RtLd4<T>::load(hr + k);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (e0 + j < outputs) {
                        const float4 wv = *reinterpret_cast<const float4*>(w0 + (size_t)j * width + k);
                        acc[j] = fmaf(hv.x, wv.x, acc[j]);
                        acc[j] = fmaf(hv.y, wv.y, acc[j]);
                        acc[j] = fmaf(hv.z, wv.z, acc[j]);
                        acc[j] = fmaf(hv.w, wv.w, acc[j]);
                    }
                }
            }
        } else {
            for (int k = lane; k < width; k += 32) {
                const float hv = to_f32(hr[k]);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (e0 + j < outputs) acc[j] = fmaf(hv, w0[(size_t)j * width + k], acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0 && e0 + j < outputs) s[e0 + j] = bias ? v + bias[e0 + j] : v;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    {

    __syncwarp();
    if (score_mode == 1) {
        for (int e = lane; e < outputs; e += 32) choice[e] = s[e];
    } else {
    float mx = -INFINITY;
    for (int e = lane; e < outputs; e += 32) mx = fmaxf(mx, s[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) sum += expf(s[e] - mx);
    sum = warp_sum(sum);
    for (int e = lane; e < outputs; e += 32) {
        const float p = expf(s[e] - mx) / sum;
        s[e] = p;
        choice[e] = p + (corr ? corr[e] : 0.f);
    }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = outputs / groups;
        for (int gi = lane; gi < groups; gi += 32) {
            float m = -INFINITY;
            for (int e = gi * per; e < (gi + 1) * per; ++e) m = fmaxf(m, choice[e]);
            gscore[gi] = m;
        }
        __syncwarp();
        // the best `keep` groups, one after the other; a chosen group is marked by +inf
        for (int r = 0; r < keep; ++r) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int gi = lane; gi < groups; gi += 32) {
                const float v = gscore[gi];
                if (v != INFINITY && (v > bv || (v == bv && gi < bi) || bi == 0x7fffffff)) { bv = v; bi = gi; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0 && bi != 0x7fffffff) gscore[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < outputs; e += 32)
            if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int r = 0; r < top; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < outputs; e += 32) {
            const float v = choice[e];
            if (!isnan(v) && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;              // (cannot happen with top <= the outputs that may be chosen)
        const float p = s[bi];
        total += p;
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            wts[(size_t)t * top + r] = p;
            choice[bi] = NAN;                      // taken
        }
        __syncwarp();
    }
    if (lane == 0 && score_mode == 1) {
        // the softmax over the chosen logits; the first choice is the largest
        const float z0 = wts[(size_t)t * top];
        float sum = 0.f;
        for (int r = 0; r < top; ++r) {
            const float p = expf(wts[(size_t)t * top + r] - z0);
            wts[(size_t)t * top + r] = p;
            sum += p;
        }
        const float inv = 1.f / sum;
        for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] *= inv;
    } else if (lane == 0) {
        const float inv = 1.f / (total + 1e-20f);
        for (int r = 0; r < top; ++r) wts[(size_t)t * top + r] *= inv;
    }
    __syncwarp();
    }
}

// One block: the pairs counted per expert (a pair's rank within its expert comes from the count, in shared
// memory), counts -> offsets, the pairs listed expert by expert, the tiles.  plan[0] = number of tiles.
__global__ void moe_plan_kernel(const int* __restrict__ ids, int* __restrict__ ranks, int* __restrict__ offsets,
                                int* __restrict__ pair_of, int* __restrict__ plan, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int pairs, int experts, int tile_m) {
    extern __shared__ int pl_smem[];           // counts [experts], offsets [experts + 1]
    int* cnt = pl_smem;
    int* off = pl_smem + experts;
    pdl_trigger();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    pdl_wait();
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e < experts) ranks[p] = atomicAdd(cnt + e, 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            off[e] = acc;
            offsets[e] = acc;
            const int c = cnt[e];
            for (int r = 0; r < c; r += tile_m) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = acc + r;
                ++tiles;
            }
            acc += c;
        }
        off[experts] = acc;
        offsets[experts] = acc;
        plan[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e < experts) pair_of[off[e] + ranks[p]] = p;
    }
}

// what a gated expert makes of a gate row's and an up row's product (see the top of the file)
__device__ __forceinline__ float gated_act(float g, float u, float limit, float alpha, float shift) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return g / (1.f + expf(-alpha * g)) * (u + shift);
}

// ids[t, k] = table[token[t], k], each with weight 1 / top.  A token id outside the table is a status, not a read.
__global__ void moe_table_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int vocab,
                                       int* __restrict__ ids, float* __restrict__ wts, int n, int top, int experts,
                                       int* __restrict__ status) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (p >= n * top) return;
    const int t = p / top, k = p - t * top;
    const int tok = tokens[t];
    int e = 0;
    if (tok < 0 || tok >= vocab) {
        if (status) atomicExch(status, 1);
    } else {
        e = table[(size_t)tok * top + k];
        if (e < 0 || e >= experts) {
            if (status) atomicExch(status, 1);
            e = 0;
        }
    }
    ids[p] = e;
    wts[p] = 1.f / (float)top;
}

// out rows of one tile = act(A rows x W[e]^T): A [*, K] rows gathered through `src` (pair / src_div when
// gather, else the sorted position itself), W [experts, N, K].  MODE 0 (up): out[pos, :] = relu(.)^2 in T.
// MODE 1 (down): out[pair, :] = weight[pair] * (.) in float.  MODE 2 (gate and up in one matrix, rows alternating
// gate_j, up_j): out[pos, j] = silu(gate_j) * up_j in T, out having N / 2 columns.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ A, long long a_stride, const T* __restrict__ W, const int* __restrict__ plan,
                   const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const int* __restrict__ offsets, const int* __restrict__ pair_of, const float* __restrict__ wts,
                   void* __restrict__ out, int N, int K, int top, float act_limit, float act_alpha, float act_shift) {
    __shared__ float As[MOE_TK][MOE_TM + 4];
    __shared__ float Ws[MOE_TK][MOE_TN + 4];
    __shared__ int s_src[MOE_TM], s_dst[MOE_TM];
    const int tile = blockIdx.x;
    const int c0 = blockIdx.y * MOE_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    pdl_trigger();
    pdl_wait();
    if (tile >= plan[0]) return;
    const int e = tile_expert[tile], row0 = tile_row0[tile];
    const int rows = min(MOE_TM, offsets[e + 1] - row0);
    if (threadIdx.x < MOE_TM) {
        int src = -1, dst = -1;
        if ((int)threadIdx.x < rows) {
            const int pos = row0 + threadIdx.x;
            const int pair = pair_of[pos];
            src = MODE != 1 ? pair / top : pos;
            dst = MODE != 1 ? pos : pair;
        }
        s_src[threadIdx.x] = src;
        s_dst[threadIdx.x] = dst;
    }
    __syncthreads();
    const T* We = W + (size_t)e * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        for (int idx = threadIdx.x; idx < MOE_TM * MOE_TK; idx += 256) {
            const int rr = idx / MOE_TK, kk = idx - rr * MOE_TK;
            const int src = s_src[rr], k = k0 + kk;
            As[kk][rr] = (src >= 0 && k < K) ? to_f32(A[(size_t)src * a_stride + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < MOE_TN * MOE_TK; idx += 256) {
            const int cc = idx / MOE_TK, kk = idx - cc * MOE_TK;
            const int c = c0 + cc, k = k0 + kk;
            Ws[kk][cc] = (c < N && k < K) ? to_f32(We[(size_t)c * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float aa[4] = {av.x, av.y, av.z, av.w};
            const float ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], ww[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int dst = s_dst[ty * 4 + i];
        if (dst < 0) continue;
        const float g = MODE == 1 ? wts[dst] : 1.f;
        if (MODE == 2) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int c = c0 + tx * 4 + j;
                if (c + 1 >= N) continue;
                reinterpret_cast<T*>(out)[(size_t)dst * (N >> 1) + (c >> 1)] =
                    from_f32<T>(gated_act(acc[i][j], acc[i][j + 1], act_limit, act_alpha, act_shift));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + tx * 4 + j;
                if (c >= N) continue;
                if (MODE == 0) {
                    const float r = fmaxf(acc[i][j], 0.f);
                    reinterpret_cast<T*>(out)[(size_t)dst * N + c] = from_f32<T>(r * r);
                } else {
                    reinterpret_cast<float*>(out)[(size_t)dst * N + c] = g * acc[i][j];
                }
            }
        }
    }
}

// The same tile on the tensor cores for bfloat16 (K a multiple of 8, rows 16-byte aligned): see mma_tile.cuh.
template <int MODE, int BM, int BN, int WM, int WN>
__global__ void __launch_bounds__(WM * WN * 32)
moe_grouped_mma_kernel(const __nv_bfloat16* __restrict__ A, long long a_stride, const __nv_bfloat16* __restrict__ W,
                       const int* __restrict__ plan, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                       const int* __restrict__ offsets, const int* __restrict__ pair_of, const float* __restrict__ wts,
                       void* __restrict__ out, int N, int K, int top, float act_limit, float act_alpha, float act_shift) {
    extern __shared__ __align__(128) unsigned char moe_smem[];
    using Tile = MmaTile<BM, BN, WM, WN>;
    __shared__ const __nv_bfloat16* a_rows[BM];
    __shared__ const __nv_bfloat16* w_rows[BN];
    __shared__ int s_dst[BM];
    const int tile = blockIdx.x;
    const int c0 = blockIdx.y * BN;
    pdl_trigger();
    pdl_wait();
    if (tile >= plan[0]) return;
    const int e = tile_expert[tile], row0 = tile_row0[tile];
    const int rows = min(BM, offsets[e + 1] - row0);
    const __nv_bfloat16* We = W + (size_t)e * N * K;
    for (int r = threadIdx.x; r < BN; r += Tile::THREADS) w_rows[r] = c0 + r < N ? We + (size_t)(c0 + r) * K : nullptr;
    for (int r = threadIdx.x; r < BM; r += Tile::THREADS) {
        const __nv_bfloat16* ap = nullptr;
        int dst = -1;
        if (r < rows) {
            const int pos = row0 + r;
            const int pair = pair_of[pos];
            ap = A + (size_t)(MODE != 1 ? pair / top : pos) * a_stride;
            dst = MODE != 1 ? pos : pair;
        }
        a_rows[r] = ap;
        s_dst[r] = dst;
    }
    __syncthreads();
    float acc[Tile::MI][Tile::NI][4];
    Tile::run(a_rows, w_rows, K, W, reinterpret_cast<__nv_bfloat16*>(moe_smem), acc);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp / WN, wn = warp % WN, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mi = 0; mi < Tile::MI; ++mi)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int dst = s_dst[wm * (BM / WM) + mi * 16 + g + 8 * h];
            if (dst < 0) continue;
            const float gw = MODE == 1 ? wts[dst] : 1.f;
#pragma unroll
            for (int ni = 0; ni < Tile::NI; ++ni) {
                const int c = c0 + wn * (BN / WN) + ni * 8 + 2 * t;
                const float v0 = acc[mi][ni][2 * h], v1 = acc[mi][ni][2 * h + 1];
                if (MODE == 2) {
                    // (c is even: v0 is a gate's row, v1 the up row that belongs to it)
                    if (c + 1 < N)
                        reinterpret_cast<__nv_bfloat16*>(out)[(size_t)dst * (N >> 1) + (c >> 1)] =
                            __float2bfloat16_rn(gated_act(v0, v1, act_limit, act_alpha, act_shift));
                } else if (MODE == 0) {
                    const float r0 = fmaxf(v0, 0.f), r1 = fmaxf(v1, 0.f);
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)dst * N + c;
                    if (c + 1 < N && (N & 1) == 0) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(r0 * r0, r1 * r1);
                    else {
                        if (c < N) o[0] = __float2bfloat16_rn(r0 * r0);
                        if (c + 1 < N) o[1] = __float2bfloat16_rn(r1 * r1);
                    }
                } else {
                    float* o = reinterpret_cast<float*>(out) + (size_t)dst * N + c;
                    if (c + 1 < N && (N & 1) == 0) *reinterpret_cast<float2*>(o) = make_float2(gw * v0, gw * v1);
                    else {
                        if (c < N) o[0] = gw * v0;
                        if (c + 1 < N) o[1] = gw * v1;
                    }
                }
            }
        }
}

// out[t, :] = sum over the token's choices (an expert's row of y, or weight * h for an identity expert)
// + shared[t, :] (when given), in the order of the choices.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ ids, const float* __restrict__ wts,
                                   const T* __restrict__ h, const T* __restrict__ shared, T* __restrict__ out, int n,
                                   int width, int top, int experts) {
    const int t = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (t >= n) return;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < top; ++r) {
            const size_t p = (size_t)t * top + r;
            acc += ids[p] < experts ? y[p * width + c] : wts[p] * to_f32(h[(size_t)t * width + c]);
        }
        if (shared) acc += to_f32(shared[(size_t)t * width + c]);
        out[(size_t)t * width + c] = from_f32<T>(acc);
    }
}

template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ x, T* __restrict__ out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= total) return;
    const float r = fmaxf(to_f32(x[i]), 0.f);
    out[i] = from_f32<T>(r * r);
}

// 16 bytes a thread (total a multiple of 8, both pointers 16-byte aligned)
__global__ void relu_squared_bf16x8_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, long long total8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (i >= total8) return;
    uint4 v = x[i];
    unsigned* w = reinterpret_cast<unsigned*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[k]));
        f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
        __nv_bfloat162 r = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
        w[k] = *reinterpret_cast<unsigned*>(&r);
    }
    out[i] = v;
}

VAPI_EXPORT int vapi_relu_squared(const void* x, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (dtype == VAPI_BF16 && total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0)
        return check_launch("relu_squared", launch(relu_squared_bf16x8_kernel, (int)((total / 8 + 255) / 256), 256, 0, stream,
                                                   (const uint4*)x, (uint4*)out, total / 8));
    const int blocks = (int)((total + 255) / 256);
    cudaError_t e;
    if (dtype == VAPI_F32) e = launch(relu_squared_kernel<float>, blocks, 256, 0, stream, (const float*)x, (float*)out, total);
    else if (dtype == VAPI_BF16)
        e = launch(relu_squared_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, total);
    else return fail(-2, "relu_squared: unsupported dtype %d", dtype);
    return check_launch("relu_squared", e);
}

// ids, wts, ranks: [n, top]; offsets: [experts + 1]; pair_of: [n * top];
// plan: [1]; tile_expert, tile_row0: [max_tiles] with max_tiles >= n * top / 64 + experts.
VAPI_EXPORT int vapi_moe_route(const void* h, int dtype, const float* wr, const float* corr, const float* bias,
                               int score_mode, int* ids, float* wts, int* ranks,
                               int* offsets, int* pair_of, int* plan, int* tile_expert, int* tile_row0, int n,
                               int width, int outputs, int experts, int top, int groups, int keep, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (outputs <= 0 || experts < 0 || experts > outputs || top <= 0 || top > outputs)
        return fail(-1, "moe_route: %d outputs, %d experts, top %d", outputs, experts, top);
    if (groups < 1 || outputs % groups || keep < 1 || keep > groups)
        return fail(-1, "moe_route: %d outputs in %d groups, %d kept", outputs, groups, keep);
    if ((long long)(outputs / groups) * keep < top) return fail(-1, "moe_route: %d kept groups cannot give %d choices", keep, top);
    cudaError_t e;
    const size_t smem = (size_t)(2 * outputs + groups) * sizeof(float);
    if (smem > 48 * 1024) return fail(-1, "moe_route: %d router outputs are too many", outputs);
    const int vec4 = (width % 4 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)wr & 15) == 0) ? 1 : 0;
    if (dtype == VAPI_F32)
        e = launch(moe_route_kernel<float>, n, 128, smem, stream, (const float*)h, wr, corr, bias, score_mode, ids, wts, n,
                   width, outputs, experts, top, groups, keep, vec4);
    else if (dtype == VAPI_BF16)
        e = launch(moe_route_kernel<__nv_bfloat16>, n, 128, smem, stream, (const __nv_bfloat16*)h, wr, corr, bias, score_mode, ids,
                   wts, n, width, outputs, experts, top, groups, keep, vec4);
    else
        return fail(-2, "moe_route: unsupported dtype %d", dtype);
    int rc = check_launch("moe_route", e);
    if (rc != 0 || experts == 0) return rc;
    const size_t psm = sizeof(int) * (size_t)(2 * experts + 1);
    if (psm > 48 * 1024) return fail(-1, "moe_route: %d experts are too many", experts);
    e = launch(moe_plan_kernel, 1, 1024, psm, stream, (const int*)ids, ranks, offsets, pair_of, plan, tile_expert, tile_row0,
               n * top, experts, moe_tile_rows(n * top, experts));
    return check_launch("moe_plan", e);
}

// The router-less choice: ids and weights from a table over the token ids, then the same plan.
VAPI_EXPORT int vapi_moe_table_route(const int* tokens, const int* table, int vocab, int* ids, float* wts, int* ranks,
                                     int* offsets, int* pair_of, int* plan, int* tile_expert, int* tile_row0, int n,
                                     int experts, int top, int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || vocab <= 0)
        return fail(-1, "moe_table_route: %d experts, top %d, a table of %d rows", experts, top, vocab);
    const int pairs = n * top;
    cudaError_t e = launch(moe_table_route_kernel, (pairs + 255) / 256, 256, 0, stream, tokens, table, vocab, ids, wts, n, top,
                           experts, status);
    int rc = check_launch("moe_table_route", e);
    if (rc != 0) return rc;
    const size_t psm = sizeof(int) * (size_t)(2 * experts + 1);
    if (psm > 48 * 1024) return fail(-1, "moe_table_route: %d experts are too many", experts);
    e = launch(moe_plan_kernel, 1, 1024, psm, stream, (const int*)ids, ranks, offsets, pair_of, plan, tile_expert, tile_row0,
               pairs, experts, moe_tile_rows(pairs, experts));
    return check_launch("moe_plan", e);
}

// mode 0: out = hid [n * top, N] in the activation type from A = h [n, K]; mode 1: out = y [n * top, N] float
// from A = hid [n * top, K].
VAPI_EXPORT int vapi_moe_grouped(const void* A, long long a_stride, const void* W, int dtype, const int* plan,
                                 const int* tile_expert, const int* tile_row0, const int* offsets, const int* pair_of,
                                 const float* wts, void* out, int pairs, int experts, int N, int K, int top, int mode,
                                 cudaStream_t stream, float act_limit, float act_alpha, float act_shift) {
    if (pairs <= 0 || experts <= 0) return 0;
    if (mode < 0 || mode > 2 || (mode == 2 && (N & 1))) return fail(-1, "moe_grouped: mode %d with %d output rows", mode, N);
    const int max_tiles = pairs / MOE_TM + experts;
    dim3 grid(max_tiles, (N + MOE_TN - 1) / MOE_TN);
    if (grid.y > 65535) return fail(-1, "moe_grouped: %d output features are too many", N);
    cudaError_t e;
    const int tile_m = moe_tile_rows(pairs, experts);
    if (dtype == VAPI_BF16 && K % 8 == 0 && a_stride % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
#define MOE_TC(M, BM_, BN_, WM_, WN_)                                                                                        \
    do {                                                                                                                     \
        using Tile = MmaTile<BM_, BN_, WM_, WN_>;                                                                            \
        auto kern = moe_grouped_mma_kernel<M, BM_, BN_, WM_, WN_>;                                                           \
        static bool attr_set = false;                                                                                        \
        if (!attr_set) {                                                                                                     \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile::SMEM) != cudaSuccess)     \
                return fail(-101, "moe_grouped: cannot reserve %zu bytes of shared memory", Tile::SMEM);                     \
            attr_set = true;                                                                                                 \
        }                                                                                                                    \
        dim3 g(pairs / BM_ + experts, (N + BN_ - 1) / BN_);                                                                  \
        e = launch(kern, g, Tile::THREADS, Tile::SMEM, stream, (const __nv_bfloat16*)A, a_stride, (const __nv_bfloat16*)W,   \
                   plan, tile_expert, tile_row0, offsets, pair_of, wts, out, N, K, top, act_limit, act_alpha, act_shift);    \
    } while (0)
        if (mode == 0) MOE_TC(0, 64, 64, 2, 2); else if (mode == 1) MOE_TC(1, 64, 64, 2, 2); else MOE_TC(2, 64, 64, 2, 2);
#undef MOE_TC
        return check_launch("moe_grouped (tensor cores)", e);
    }
    if (tile_m != MOE_TM) return fail(-1, "moe_grouped: the float kernel has tiles of %d rows", MOE_TM);
#define MOE_GO(T, M)                                                                                                         \
    e = launch(moe_grouped_kernel<T, M>, grid, 256, 0, stream, (const T*)A, a_stride, (const T*)W, plan, tile_expert,         \
               tile_row0, offsets, pair_of, wts, out, N, K, top, act_limit, act_alpha, act_shift)
    if (dtype == VAPI_F32) { if (mode == 0) MOE_GO(float, 0); else if (mode == 1) MOE_GO(float, 1); else MOE_GO(float, 2); }
    else if (dtype == VAPI_BF16) {
        if (mode == 0) MOE_GO(__nv_bfloat16, 0); else if (mode == 1) MOE_GO(__nv_bfloat16, 1); else MOE_GO(__nv_bfloat16, 2);
    }
    else return fail(-2, "moe_grouped: unsupported dtype %d", dtype);
#undef MOE_GO
    return check_launch("moe_grouped", e);
}

VAPI_EXPORT int vapi_moe_combine(const float* y, const int* ids, const float* wts, const void* h, const void* shared,
                                 void* out, int dtype, int n, int width, int top, int experts, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(moe_combine_kernel<float>, n, threads, 0, stream, y, ids, wts, (const float*)h, (const float*)shared,
                   (float*)out, n, width, top, experts);
    else if (dtype == VAPI_BF16)
        e = launch(moe_combine_kernel<__nv_bfloat16>, n, threads, 0, stream, y, ids, wts, (const __nv_bfloat16*)h,
                   (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, n, width, top, experts);
    else
        return fail(-2, "moe_combine: unsupported dtype %d", dtype);
    return check_launch("moe_combine", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
