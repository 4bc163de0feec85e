// Tensor-core attention over a shared cache row (latent attention), bfloat16.
//
// Every token has ONE cached row of dk elements, [latent (dv) | rotated key part (dk - dv)], which all heads read: a
// score is scale * q . row over the whole row and a head's output is the softmax-weighted sum of the rows' first dv
// elements.  So a key tile in shared memory is the B operand of both products: of Q.K^T as it lies ([key][element]:
// ldmatrix), and of P.V through ldmatrix.trans over its first dv columns.  It is fetched once.
//
// Work decomposition as in the other flash kernels of the package: the rows of one sequence are its (query token, head)
// pairs (one kv head: all heads of a token share the keys), cut into tiles of 64; a block of four warps takes one tile,
// a warp 16 rows of it; keys are walked in tiles of 64 through two shared-memory stages of 16-byte cp.async copies (rows
// padded by 16 bytes, which makes ldmatrix conflict-free when dk is a multiple of 16); keys no row can see are stored as
// zeros, so uninitialised cache memory never reaches the arithmetic.  mma.sync m16n8k16, float accumulators; scores,
// mask, running maximum and sum in float registers; P is rounded to bfloat16 only as the operand of P.V.  With splits >
// 1 the key tiles are divided among blocks that leave partial results for the fixed-order combine of
// attention_masked.cu.
//
// dk and dv multiples of 16, dv <= dk, dv <= 8 * NTV (the accumulator's registers are sized by the template; widths
// are run-time values below that).
#pragma once
#include "common.cuh"
#include "attention_mma.cuh"

namespace vapi {

__device__ __forceinline__ void lf_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lf_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}

constexpr int LF_ROWS = 64;
constexpr int LF_BK = 64;
constexpr int LF_THREADS = 128;

template <int NTV>
__global__ void __launch_bounds__(LF_THREADS)
latent_flash_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, const __nv_bfloat16* __restrict__ cache,
                    const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_q,
                    const int* __restrict__ seqlens_k, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int nh, int dk, int dv, int page_size, int num_pages, float scale,
                    int splits, int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char lf_smem[];
    const int ldk = dk + 8;                                            // elements; rows stay 16-byte aligned
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(lf_smem);     // [LF_ROWS][ldk]
    __nv_bfloat16* sK = sQ + LF_ROWS * ldk;                            // [2][LF_BK][ldk]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int s = blockIdx.y / splits, sp = blockIdx.y - s * splits;
    pdl_trigger();
    const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0, klen = seqlens_k[s];
    const int rows_total = qlen * nh;
    // row tiles late in a sequence see the most keys: hand them out first
    const int tile_start = ((int)gridDim.x - 1 - (int)blockIdx.x) * LF_ROWS;
    if (tile_start >= rows_total) {
        pdl_wait();
        return;
    }
    const int last_row = min(rows_total, tile_start + LF_ROWS) - 1;
    const int base_pos = klen - qlen;
    const int p_max = base_pos + last_row / nh;
    const int ntiles_all = p_max / LF_BK + 1;
    const int per = (ntiles_all + splits - 1) / splits;
    const int it_begin = sp * per, it_end = min(ntiles_all, it_begin + per);
    const int* bt = block_table + (size_t)s * table_stride;
    const int cpr = dk >> 3;                                           // 16-byte chunks in a row
    pdl_wait();

    // ---- the queries of the tile, once
    for (int idx = threadIdx.x; idx < LF_ROWS * cpr; idx += LF_THREADS) {
        const int lr = idx / cpr, c = idx - lr * cpr;
        const int rr = tile_start + lr;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (rr < rows_total) {
            const int tok = rr / nh, h = rr - tok * nh;
            v = *reinterpret_cast<const uint4*>(q + (size_t)(q0 + tok) * q_row_stride + (size_t)h * dk + c * 8);
        }
        *reinterpret_cast<uint4*>(sQ + lr * ldk + c * 8) = v;
    }

    auto load_keys = [&](int it, int stage) {
        __nv_bfloat16* dst = sK + (size_t)stage * LF_BK * ldk;
        const int j0 = it * LF_BK;
        // a warp takes every fourth row, its lanes the row's 16-byte chunks: one page lookup a row
        for (int jj = warp; jj < LF_BK; jj += LF_THREADS / 32) {
            const int j = j0 + jj;
            __nv_bfloat16* d = dst + jj * ldk;
            bool ok = j <= p_max && j < klen;
            const __nv_bfloat16* src = cache;
            if (ok) {
                const int pi = j / page_size;
                const int page = bt[pi];
                if (page < 0 || page >= num_pages) {
                    if (lane == 0 && status) atomicExch(status, 4);
                    ok = false;
                } else {
                    src = cache + ((size_t)page * page_size + (j - pi * page_size)) * dk;
                }
            }
            if (ok) {
                for (int c = lane; c < cpr; c += 32) cp_async_16(d + c * 8, src + c * 8, 16);
            } else {
                for (int c = lane; c < cpr; c += 32) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    // rows of this thread: gq and gq + 8 of the warp's sixteen
    int row_pos[2];
    bool row_ok[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int rr = tile_start + warp * 16 + gq + 8 * h2;
        row_ok[h2] = rr < rows_total;
        row_pos[h2] = base_pos + (row_ok[h2] ? rr / nh : 0);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[NTV][4];
#pragma unroll
    for (int i = 0; i < NTV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    const int ksteps = dk >> 4, ntv = dv >> 3;
    // this lane's ldmatrix addresses (bytes in shared memory), to which the loops add constants
    const unsigned row_bytes = (unsigned)ldk * 2u;
    const unsigned aq = (unsigned)__cvta_generic_to_shared(sQ) + (unsigned)(warp * 16 + (lane & 15)) * row_bytes + (unsigned)(lane >> 4) * 16u;
    const unsigned ak0 = (unsigned)__cvta_generic_to_shared(sK) + (unsigned)((lane & 7) + (lane >> 4) * 8) * row_bytes + (unsigned)((lane >> 3) & 1) * 16u;
    const unsigned av0 = (unsigned)__cvta_generic_to_shared(sK) + (unsigned)((lane & 7) + ((lane >> 3) & 1) * 8) * row_bytes + (unsigned)(lane >> 4) * 16u;
    const unsigned stage_bytes = (unsigned)LF_BK * row_bytes;
    const float scale2 = scale * 1.4426950408889634f;          // scores in units of log 2, so that exp is exp2
    const int warp_p_min = base_pos + min(tile_start + warp * 16, rows_total - 1) / nh;

    if (it_begin < it_end) load_keys(it_begin, 0);
    cp_async_commit();
    for (int it = it_begin; it < it_end; ++it) {
        const int stage = (it - it_begin) & 1;
        if (it + 1 < it_end) load_keys(it + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned ak = ak0 + (unsigned)stage * stage_bytes, av = av0 + (unsigned)stage * stage_bytes;

        // ---- scores of 16 rows x 32 keys
        float sc[LF_BK / 8][4];
#pragma unroll
        for (int i = 0; i < LF_BK / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[i][e] = 0.f;
        for (int ks = 0; ks < ksteps; ++ks) {
            unsigned a[4];
            lf_ldmatrix_x4(a[0], a[1], a[2], a[3], aq + (unsigned)ks * 32u);
#pragma unroll
            for (int np = 0; np < LF_BK / 16; ++np) {
                unsigned b0, b1, b2, b3;
                lf_ldmatrix_x4(b0, b1, b2, b3, ak + (unsigned)np * 16u * row_bytes + (unsigned)ks * 32u);
                mma_bf16_16816(sc[2 * np], a, b0, b1);
                mma_bf16_16816(sc[2 * np + 1], a, b2, b3);
            }
        }
        // ---- mask, running maximum and sum
        float mx[2] = {-INFINITY, -INFINITY};
        if (it * LF_BK + LF_BK - 1 <= warp_p_min && row_ok[1]) {
            // every key of the tile lies at or before every row of the warp: nothing to mask
#pragma unroll
            for (int i = 0; i < LF_BK / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sc[i][e] *= scale2;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sc[i][e]);
                }
        } else {
#pragma unroll
            for (int i = 0; i < LF_BK / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h2 = e >> 1;
                    const int j = it * LF_BK + i * 8 + 2 * tq + (e & 1);
                    const bool vis = row_ok[h2] && j <= row_pos[h2] && j < klen;
                    sc[i][e] = vis ? sc[i][e] * scale2 : -INFINITY;
                    mx[h2] = fmaxf(mx[h2], sc[i][e]);
                }
        }
        float alpha[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
            const float m_new = fmaxf(m[h2], mx[h2]);
            alpha[h2] = m_new == -INFINITY ? 1.f : exp2f(m[h2] - m_new);
            m[h2] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        unsigned pa[LF_BK / 16][4];
#pragma unroll
        for (int i = 0; i < LF_BK / 8; ++i) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h2 = e >> 1;
                p[e] = sc[i][e] == -INFINITY ? 0.f : exp2f(sc[i][e] - m[h2]);
                rs[h2] += p[e];
            }
            pa[i >> 1][(i & 1) * 2] = pack_bf16(p[0], p[1]);
            pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            rs[h2] += __shfl_xor_sync(0xffffffffu, rs[h2], 1);
            rs[h2] += __shfl_xor_sync(0xffffffffu, rs[h2], 2);
            l[h2] = l[h2] * alpha[h2] + rs[h2];
        }
#pragma unroll
        for (int i = 0; i < NTV; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        // ---- P.V over the tile's first dv columns
#pragma unroll
        for (int kk = 0; kk < LF_BK / 16; ++kk) {
#pragma unroll
            for (int nv = 0; nv < NTV / 2; ++nv) {
                if (2 * nv < ntv) {
                    unsigned b0, b1, b2, b3;
                    lf_ldmatrix_x4_trans(b0, b1, b2, b3, av + (unsigned)kk * 16u * row_bytes + (unsigned)nv * 32u);
                    mma_bf16_16816(o[2 * nv], pa[kk], b0, b1);
                    mma_bf16_16816(o[2 * nv + 1], pa[kk], b2, b3);
                }
            }
        }
        __syncthreads();            // the stage is refilled by the next iteration's copies
    }
    cp_async_wait<0>();

    // ---- out
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (!row_ok[h2]) continue;
        const int rr = tile_start + warp * 16 + gq + 8 * h2;
        const int tok = rr / nh, h = rr - tok * nh;
        const size_t grow = (size_t)(q0 + tok) * nh + h;
        if (splits == 1) {
            const float inv = l[h2] > 0.f ? 1.f / l[h2] : 0.f;
#pragma unroll
            for (int i = 0; i < NTV; ++i) {
                if (i < ntv) {
                    *reinterpret_cast<__nv_bfloat162*>(out + grow * dv + i * 8 + 2 * tq) =
                        __floats2bfloat162_rn(o[i][2 * h2] * inv, o[i][2 * h2 + 1] * inv);
                }
            }
        } else {
            float* po = part_o + (grow * splits + sp) * (size_t)dv;
#pragma unroll
            for (int i = 0; i < NTV; ++i) {
                if (i < ntv) *reinterpret_cast<float2*>(po + i * 8 + 2 * tq) = make_float2(o[i][2 * h2], o[i][2 * h2 + 1]);
            }
            if (tq == 0) {
                part_ml[(grow * splits + sp) * 2] = m[h2] * 0.6931471805599453f;      // back to natural units for the combine
                part_ml[(grow * splits + sp) * 2 + 1] = l[h2];
            }
        }
    }
}

inline bool latent_flash_applies(int dk, int dv, long long q_row_stride, const void* q, const void* cache, const void* out) {
    return dk % 16 == 0 && dv % 16 == 0 && dv <= dk && dv <= 256 && dk <= 640 && q_row_stride % 8 == 0 &&
           (((uintptr_t)q | (uintptr_t)cache) & 15) == 0 && ((uintptr_t)out & 3) == 0;
}

// the kernel alone: with splits > 1 the caller combines the partial results
static int launch_latent_flash(const void* q, long long q_row_stride, const void* cache, const int* block_table, int table_stride,
                               const int* cu_q, const int* seqlens_k, void* out, float* part_o, float* part_ml, int num_seqs,
                               int max_q, int nh, int dk, int dv, int page_size, int num_pages, float scale, int splits,
                               int* status, cudaStream_t stream) {
    const size_t smem = (size_t)(LF_ROWS + 2 * LF_BK) * (dk + 8) * sizeof(__nv_bfloat16);
    const int tiles = (int)(((long long)max_q * nh + LF_ROWS - 1) / LF_ROWS);
    if ((long long)num_seqs * splits > 65535) return fail(-1, "latent attention: %d sequences in %d splits", num_seqs, splits);
    dim3 grid(tiles, num_seqs * splits);
    cudaError_t e;
#define LF_GO(NTV_)                                                                                                            \
    do {                                                                                                                       \
        auto kern = latent_flash_kernel<NTV_>;                                                                                 \
        static size_t allowed = 0;                                                                                             \
        if (smem > 48 * 1024 && smem > allowed) {                                                                              \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)             \
                return fail(-3, "latent attention: %zu bytes of shared memory are not available", smem);                       \
            allowed = smem;                                                                                                    \
        }                                                                                                                      \
        e = launch(kern, grid, LF_THREADS, smem, stream, (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)cache,   \
                   block_table, table_stride, cu_q, seqlens_k, (__nv_bfloat16*)out, part_o, part_ml, nh, dk, dv, page_size,    \
                   num_pages, scale, splits, status);                                                                          \
    } while (0)
    if (dv <= 64) LF_GO(8);
    else if (dv <= 128) LF_GO(16);
    else LF_GO(32);
#undef LF_GO
    return check_launch("latent attention (tensor cores)", e);
}

}  // namespace vapi
