// Paged grouped-query attention in its most general form: keys of width dk and values of width
// dv, a sliding window and / or a chunked mask, a learned sink per head in the softmax's
// denominator, and a gate per (token, head) on the way out.  All arithmetic is float; storage is
// float or bfloat16.  It serves both number formats for mixers whose shape the specialised
// kernels of attention.cu do not take.
//
// A sequence brings len_q queries over len_k keys; query j sits at position p = len_k - len_q + j
// and sees key i iff  i <= p,  (i > p - window  or  i < keep)  (window > 0; keep: the first tokens of a
// sequence that a window never leaves behind)  and  floor(i / chunk) = floor(p / chunk)
// (chunk > 0; chunks are counted from position 0 of the sequence).  score = scale * q.k; the
// softmax's denominator also holds exp(sink_h) when sinks are given (no key, no value, unscaled);
// head h's output is multiplied by sigmoid(gate[token, h]) when a gate is given.
//
// A cache page holds the keys [nkv, page_size, dk] and then the values [nkv, page_size, dv].  With `shared_kv` a
// page holds the key rows alone and a key's value is the first dv elements of its own row (latent attention: the
// cached latent is both, and the rotated key part follows it in the row); dv <= dk then.
//
// bfloat16 with `shared_kv` and widths that are multiples of 16 (values up to 256) runs on the tensor-core kernel of
// attention_latent.cuh.  bfloat16 with keys and values of one width, 64 or 128, and pages of a multiple of 64 tokens runs on
// the tensor cores: the flash kernel of attention_mma.cuh (four warps for prompt portions, one warp
// per 16 rows and split keys for decode steps) and, for prompt portions of 64 tokens and more at
// width 64, the tcgen05 kernel of attention_tc.cuh; both take the mask, the sink and the gate as
// parameters.  Everything else (float32, unlike widths, other sizes) runs on the kernel below.
//
// Work decomposition as in the general kernel of attention.cu: for one (sequence, kv head) the
// rows are the pairs (query token, q head of the group), cut into tiles of 16; a block of four
// warps takes one tile and walks the keys in tiles of 32; warp w owns rows w, w+4, w+8, w+12.
// With splits > 1 the key tiles are divided among blocks that leave partial results, combined by
// a second kernel in a fixed order; the sink is counted by the first split.
#include "common.cuh"
#include "attention_mma.cuh"
#include "attention_tc.cuh"
#include "attention_latent.cuh"

using namespace vapi;

constexpr int MA_ROWS = 16;
constexpr int MA_BK = 32;
constexpr int MA_WARPS = 4;
constexpr int MA_RPW = MA_ROWS / MA_WARPS;

template <typename T> struct Ld4;
template <> struct Ld4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Ld4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(fa.x, fa.y, fb.x, fb.y);
    }
};

__device__ __forceinline__ bool ma_visible(int j, int p, int klen, int window, int chunk, int keep) {
    return j <= p && j < klen && (window <= 0 || j > p - window || j < keep) && (chunk <= 0 || j >= (p / chunk) * chunk);
}

template <typename T, int DVMAX>
__global__ void __launch_bounds__(MA_WARPS * 32)
masked_attention_kernel(const T* __restrict__ q, long long q_row_stride, const T* __restrict__ cache,
                        const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ seqlens_k, const float* __restrict__ sinks,
                        const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv, int dk, int dv,
                        int page_size, int num_pages, float scale, int window, int chunk, int splits,
                        int* __restrict__ status, int keep, int shared_kv) {
    constexpr int DPL = DVMAX / 32;
    extern __shared__ __align__(16) float smem[];
    const int ldk = dk + 4, ldv = dv + 4;
    float* Qs = smem;                      // [MA_ROWS][ldk]
    float* Ks = Qs + MA_ROWS * ldk;        // [MA_BK][ldk]
    float* Vs = Ks + MA_BK * ldk;          // [MA_BK][ldv]
    float* Ps = Vs + MA_BK * ldv;          // [MA_WARPS][MA_RPW][MA_BK]
    const float* Vr = shared_kv ? Ks : Vs;  // where a key tile's values are read
    const int ldr = shared_kv ? ldk : ldv;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.z / splits, sp = blockIdx.z - s * splits;
    const int g = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0, klen = seqlens_k[s];
    const int n_rep = nh / nkv;
    const int rows_total = qlen * n_rep;
    const int tile_start = blockIdx.x * MA_ROWS;
    if (tile_start >= rows_total) return;
    const int last_row = min(rows_total, tile_start + MA_ROWS) - 1;
    const int base_pos = klen - qlen;
    const int p_min = base_pos + tile_start / n_rep;
    const int p_max = base_pos + last_row / n_rep;
    const int chunk_lo = chunk > 0 ? (p_min / chunk) * chunk : 0;
    int key_lo = chunk_lo;
    if (window > 0) key_lo = max(key_lo, p_min - window + 1);
    const int kt_lo = key_lo / MA_BK, kt_hi = p_max / MA_BK;
    // kept first tokens that the window has left behind: their tiles come before the window's
    const int keep_hi = (window > 0 && keep > 0) ? min(keep, key_lo) : 0;
    const int kf_lo = chunk_lo / MA_BK;
    const int n_first = keep_hi > chunk_lo ? max(0, min((keep_hi + MA_BK - 1) / MA_BK, kt_lo) - kf_lo) : 0;
    const int nt = n_first + kt_hi - kt_lo + 1;
    const int per = (nt + splits - 1) / splits;
    const int it_begin = sp * per;
    const int it_end = min(nt, it_begin + per);
    const size_t page_elems = (size_t)nkv * page_size * (shared_kv ? dk : dk + dv);
    const size_t v_base = (size_t)nkv * page_size * dk;

    for (int idx = threadIdx.x; idx < MA_ROWS * (dk / 4); idx += blockDim.x) {
        const int lr = idx / (dk / 4), c4 = idx - lr * (dk / 4);
        const int rr = tile_start + lr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rr < rows_total) {
            const int tok = rr / n_rep, h = g * n_rep + (rr - tok * n_rep);
            v = Ld4<T>::load(q + (size_t)(q0 + tok) * q_row_stride + (size_t)h * dk + c4 * 4);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
        }
        *reinterpret_cast<float4*>(Qs + lr * ldk + c4 * 4) = v;
    }

    int row_pos[MA_RPW];
    bool row_ok[MA_RPW];
    float m[MA_RPW], l[MA_RPW], acc[MA_RPW][DPL];
#pragma unroll
    for (int a = 0; a < MA_RPW; ++a) {
        const int rr = tile_start + warp + MA_WARPS * a;
        row_ok[a] = rr < rows_total;
        row_pos[a] = base_pos + (row_ok[a] ? rr / n_rep : 0);
        m[a] = -INFINITY;
        l[a] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[a][c] = 0.f;
    }

    const int* bt = block_table + (size_t)s * table_stride;
    for (int it = it_begin; it < it_end; ++it) {
        const int kt = it < n_first ? kf_lo + it : kt_lo + (it - n_first);
        __syncthreads();
        for (int idx = threadIdx.x; idx < MA_BK * (dk / 4); idx += blockDim.x) {
            const int jj = idx / (dk / 4), c4 = idx - jj * (dk / 4);
            const int j = kt * MA_BK + jj;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((j >= key_lo || (j < keep_hi && j >= chunk_lo)) && j <= p_max && j < klen) {
                const int page = bt[j / page_size];
                if (page < 0 || page >= num_pages) {
                    if (status) atomicExch(status, 4);
                } else {
                    kv = Ld4<T>::load(cache + (size_t)page * page_elems + ((size_t)g * page_size + (j % page_size)) * dk + c4 * 4);
                }
            }
            *reinterpret_cast<float4*>(Ks + jj * ldk + c4 * 4) = kv;
        }
        for (int idx = threadIdx.x; idx < (shared_kv ? 0 : MA_BK * (dv / 4)); idx += blockDim.x) {
            const int jj = idx / (dv / 4), c4 = idx - jj * (dv / 4);
            const int j = kt * MA_BK + jj;
            float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((j >= key_lo || (j < keep_hi && j >= chunk_lo)) && j <= p_max && j < klen) {
                const int page = bt[j / page_size];
                if (page >= 0 && page < num_pages)
                    vv = Ld4<T>::load(cache + (size_t)page * page_elems + v_base + ((size_t)g * page_size + (j % page_size)) * dv + c4 * 4);
            }
            *reinterpret_cast<float4*>(Vs + jj * ldv + c4 * 4) = vv;
        }
        __syncthreads();

        float sc[MA_RPW];
#pragma unroll
        for (int a = 0; a < MA_RPW; ++a) sc[a] = 0.f;
        const float4* k4 = reinterpret_cast<const float4*>(Ks + lane * ldk);
        for (int c4 = 0; c4 < dk / 4; ++c4) {
            const float4 kv = k4[c4];
#pragma unroll
            for (int a = 0; a < MA_RPW; ++a) {
                if (!row_ok[a]) continue;
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + MA_WARPS * a) * ldk + c4 * 4);
                sc[a] = fmaf(qv.x, kv.x, sc[a]);
                sc[a] = fmaf(qv.y, kv.y, sc[a]);
                sc[a] = fmaf(qv.z, kv.z, sc[a]);
                sc[a] = fmaf(qv.w, kv.w, sc[a]);
            }
        }
        const int j = kt * MA_BK + lane;
        float* pw = Ps + (warp * MA_RPW) * MA_BK;
#pragma unroll
        for (int a = 0; a < MA_RPW; ++a) {
            if (!row_ok[a]) continue;
            const bool vis = ma_visible(j, row_pos[a], klen, window, chunk, keep);
            const float sv = vis ? sc[a] : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(sv));
            float p = 0.f, alpha = 1.f;
            if (m_new != -INFINITY) {
                alpha = expf(m[a] - m_new);
                p = vis ? expf(sv - m_new) : 0.f;
            }
            l[a] = l[a] * alpha + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[a][c] *= alpha;
            pw[a * MA_BK + lane] = p;
        }
        __syncwarp();
        for (int jj = 0; jj < MA_BK; ++jj) {
            float vcol[DPL];
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                vcol[c] = col < dv ? Vr[jj * ldr + col] : 0.f;
            }
#pragma unroll
            for (int a = 0; a < MA_RPW; ++a) {
                if (!row_ok[a]) continue;
                const float p = pw[a * MA_BK + jj];
#pragma unroll
                for (int c = 0; c < DPL; ++c) acc[a][c] = fmaf(p, vcol[c], acc[a][c]);
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int a = 0; a < MA_RPW; ++a) {
        if (!row_ok[a]) continue;
        const int rr = tile_start + warp + MA_WARPS * a;
        const int tok = rr / n_rep, h = g * n_rep + (rr - tok * n_rep);
        const size_t grow = (size_t)(q0 + tok) * nh + h;
        if (sinks && sp == 0) {
            // the sink joins as one more term of the denominator, with no value
            const float sk = sinks[h];
            const float m_new = fmaxf(m[a], sk);
            const float alpha = m[a] == -INFINITY ? 0.f : expf(m[a] - m_new);
            l[a] = l[a] * alpha + expf(sk - m_new);
            m[a] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[a][c] *= alpha;
        }
        if (splits == 1) {
            float inv = l[a] > 0.f ? 1.f / l[a] : 0.f;
            if (gate) inv *= 1.f / (1.f + expf(-to_f32(gate[(size_t)(q0 + tok) * gate_stride + h])));
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                if (col < dv) out[grow * dv + col] = from_f32<T>(acc[a][c] * inv);
            }
        } else {
            float* po = part_o + (grow * splits + sp) * (size_t)dv;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int col = lane + 32 * c;
                if (col < dv) po[col] = acc[a][c];
            }
            if (lane == 0) {
                part_ml[(grow * splits + sp) * 2] = m[a];
                part_ml[(grow * splits + sp) * 2 + 1] = l[a];
            }
        }
    }
}

// Partial results of `splits` (at most 32) blocks combined in split order: one warp per (token, head).
template <typename T>
__global__ void masked_attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                                                long long rows, int nh, int dv, int splits) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    if (row >= rows) return;
    float ms = -INFINITY, ls = 0.f;
    if (lane < splits) {
        ms = part_ml[(row * splits + lane) * 2];
        ls = part_ml[(row * splits + lane) * 2 + 1];
    }
    const float mx = warp_max(ms);
    const float w = ms == -INFINITY ? 0.f : expf(ms - mx);
    float lsum = 0.f;
    for (int sp = 0; sp < splits; ++sp) lsum += __shfl_sync(0xffffffffu, ls * w, sp);
    float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    if (gate) {
        const long long tok = row / nh;
        const int h = (int)(row - tok * nh);
        inv *= 1.f / (1.f + expf(-to_f32(gate[(size_t)tok * gate_stride + h])));
    }
    for (int c0 = 0; c0 < dv; c0 += 32) {
        const int col = c0 + lane;
        float o = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
            const float ws = __shfl_sync(0xffffffffu, w, sp);
            const float v = col < dv ? part_o[(row * splits + sp) * (size_t)dv + col] : 0.f;
            o += v * ws;
        }
        if (col < dv) out[row * dv + col] = from_f32<T>(o * inv);
    }
}

template <typename T, int DVMAX>
static int launch_masked(const void* q, long long q_row_stride, const void* cache, const int* block_table,
                         int table_stride, const int* cu_q, const int* seqlens_k, const float* sinks,
                         const void* gate, long long gate_stride, void* out, float* part_o, float* part_ml, int n,
                         int num_seqs, int max_q, int nh, int nkv, int dk, int dv, int page_size, int num_pages,
                         float scale, int window, int chunk, int splits, int* status, cudaStream_t stream, int keep,
                         int shared_kv) {
    const int n_rep = nh / nkv;
    const int tiles = (max_q * n_rep + MA_ROWS - 1) / MA_ROWS;
    const size_t smem = sizeof(float) * ((size_t)(MA_ROWS + MA_BK) * (dk + 4) + (size_t)MA_BK * (dv + 4) +
                                         (size_t)MA_WARPS * MA_RPW * MA_BK);
    auto kern = masked_attention_kernel<T, DVMAX>;
    static size_t allowed = 0;
    if (smem > 227 * 1024) return fail(-3, "masked_attention: heads of %d/%d need %zu bytes of shared memory", dk, dv, smem);
    if (smem > 48 * 1024 && smem > allowed) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail(-3, "masked_attention: %zu bytes of shared memory are not available", smem);
        allowed = smem;
    }
    dim3 grid(tiles, nkv, num_seqs * splits);
    cudaError_t e = launch(kern, grid, MA_WARPS * 32, smem, stream, (const T*)q, q_row_stride, (const T*)cache, block_table,
                           table_stride, cu_q, seqlens_k, sinks, (const T*)gate, gate_stride, (T*)out, part_o, part_ml, nh, nkv,
                           dk, dv, page_size, num_pages, scale, window, chunk, splits, status, keep, shared_kv);
    int rc = check_launch("masked_attention", e);
    if (rc != 0 || splits == 1) return rc;
    const long long rows = (long long)n * nh;
    e = launch(masked_attention_combine_kernel<T>, (int)((rows + 3) / 4), 128, 0, stream, (const float*)part_o,
               (const float*)part_ml, (const T*)gate, gate_stride, (T*)out, rows, nh, dv, splits);
    return check_launch("masked_attention_combine", e);
}

VAPI_EXPORT int vapi_masked_attention(const void* q, long long q_row_stride, const void* cache, int dtype,
                                      const int* block_table, int table_stride, const int* cu_q,
                                      const int* seqlens_k, const float* sinks, const void* gate,
                                      long long gate_stride, void* out, float* part_o, float* part_ml, int n,
                                      int num_seqs, int max_q, int nh, int nkv, int dk, int dv, int page_size,
                                      int num_pages, float scale, int window, int chunk, int splits, int* status,
                                      cudaStream_t stream, int keep, int shared_kv) {
    if (n <= 0 || num_seqs <= 0) return 0;
    if (shared_kv && dv > dk) return fail(-1, "masked_attention: values of %d inside key rows of %d", dv, dk);
    if (keep < 0) return fail(-1, "masked_attention: %d kept first tokens", keep);
    if (window <= 0) keep = 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv) return fail(-1, "masked_attention: %d heads over %d kv heads", nh, nkv);
    if (dk <= 0 || dk % 4 || dv <= 0 || dv % 4 || dv > 512 || dk > 640)
        return fail(-1, "masked_attention: head sizes %d/%d must be multiples of 4 (keys up to 640, values up to 512)", dk, dv);
    if (q_row_stride % 4) return fail(-1, "masked_attention: the query row stride %lld must be a multiple of 4", q_row_stride);
    if (splits < 1 || splits > 32) return fail(-1, "masked_attention: %d splits", splits);
    if (splits > 1 && (!part_o || !part_ml)) return fail(-1, "masked_attention: splits need scratch buffers");
    if (page_size <= 0 || num_pages <= 0) return fail(-1, "masked_attention: no pages");
    if (!shared_kv && dtype == VAPI_BF16 && dk == dv && (dk == 64 || dk == 128) && page_size % FA_BK == 0 && q_row_stride % 2 == 0 &&
        nkv <= 65535 && (long long)num_seqs * splits <= 65535) {
        // the cache page is [2][nkv][page_size][d] when keys and values have one width: the layout of the fast kernels
        int rc;
        const bool tc_ok = dk == FT_HD && splits == 1 && q_row_stride % 8 == 0 && scale > 0.f && max_q >= FT_AUTO_MAX_Q &&
                           ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0;
        if (tc_ok) {
            const int min_q = num_seqs == 1 ? 1 : FT_MIN_Q;
            rc = launch_flash_tc(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, num_seqs, max_q, nh,
                                 nkv, page_size, num_pages, scale, window, min_q, status, stream, chunk, sinks, gate, gate_stride, keep);
            if (rc != 0 || min_q == 1) return rc;
            return launch_flash<64, 4, 3>(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                          num_seqs, FT_MIN_Q - 1, nh, nkv, page_size, num_pages, scale, window, 1, status, stream,
                                          FT_MIN_Q, 0, chunk, sinks, gate, gate_stride, keep);
        }
        const bool few_rows = (long long)max_q * (nh / nkv) <= 16;
#define MA_FLASH(HD, NW)                                                                                                      \
    rc = launch_flash<HD, NW, 3>(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,    \
                                 num_seqs, max_q, nh, nkv, page_size, num_pages, scale, window, splits, status, stream, 0, 0, \
                                 chunk, sinks, gate, gate_stride, keep)
        if (dk == 64) { if (few_rows) MA_FLASH(64, 1); else MA_FLASH(64, 4); }
        else          { if (few_rows) MA_FLASH(128, 1); else MA_FLASH(128, 4); }
#undef MA_FLASH
        if (rc != 0 || splits == 1) return rc;
        const long long rows = (long long)n * nh;
        return check_launch("masked_attention_combine",
                            launch(masked_attention_combine_kernel<__nv_bfloat16>, (int)((rows + 3) / 4), 128, 0, stream,
                                   (const float*)part_o, (const float*)part_ml, (const __nv_bfloat16*)gate, gate_stride,
                                   (__nv_bfloat16*)out, rows, nh, dv, splits));
    }
    if (shared_kv && dtype == VAPI_BF16 && !sinks && !gate && window <= 0 && chunk <= 0 &&
        latent_flash_applies(dk, dv, q_row_stride, q, cache, out)) {
        // one cached row per token that is key and value at once: the tensor-core kernel of attention_latent.cuh
        int rc = launch_latent_flash(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, out, part_o, part_ml,
                                     num_seqs, max_q, nh, dk, dv, page_size, num_pages, scale, splits, status, stream);
        if (rc != 0 || splits == 1) return rc;
        const long long rows = (long long)n * nh;
        return check_launch("masked_attention_combine",
                            launch(masked_attention_combine_kernel<__nv_bfloat16>, (int)((rows + 3) / 4), 128, 0, stream,
                                   (const float*)part_o, (const float*)part_ml, (const __nv_bfloat16*)nullptr, (long long)0,
                                   (__nv_bfloat16*)out, rows, nh, dv, splits));
    }
#define MA_GO(T, DV) return launch_masked<T, DV>(q, q_row_stride, cache, block_table, table_stride, cu_q, seqlens_k, sinks, gate, \
                                                 gate_stride, out, part_o, part_ml, n, num_seqs, max_q, nh, nkv, dk, dv,         \
                                                 page_size, num_pages, scale, window, chunk, splits, status, stream, keep,  \
                                                 shared_kv)
    if (dtype == VAPI_F32) {
        if (dv <= 64) MA_GO(float, 64);
        if (dv <= 128) MA_GO(float, 128);
        if (dv <= 256) MA_GO(float, 256);
        MA_GO(float, 512);
    } else if (dtype == VAPI_BF16) {
        if (dv <= 64) MA_GO(__nv_bfloat16, 64);
        if (dv <= 128) MA_GO(__nv_bfloat16, 128);
        if (dv <= 256) MA_GO(__nv_bfloat16, 256);
        MA_GO(__nv_bfloat16, 512);
    }
#undef MA_GO
    return fail(-2, "masked_attention: unsupported dtype %d", dtype);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
