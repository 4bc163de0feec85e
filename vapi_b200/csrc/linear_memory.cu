// Mixers whose state is a matrix per head that every token decays and adds an outer product to:
//
//   matrix memory (mLSTM), per head, with log gates li (input) and lf (forget) and a running maximum m:
//       m' = max(lf + m, li);  keep = exp(lf + m - m');  take = exp(li - m')
//       S <- keep S + take k v^T;   n <- keep n + take k;   o = S^T q / (max(|n . q|, exp(-m')) + floor_eps)
//       li = cap tanh((a_i + b_i) / cap),   lf = logsigmoid(cap tanh((a_f + b_f) / cap))
//   gated linear attention, per head, with a decay per key channel:
//       S <- diag(alpha) S + k v^T;   o = S^T q;   alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau)
//
// q is multiplied by `q_scale` on its way in.  S is [rows, cols] (key size x value size), float, in the
// request's state slot, stored column by column ([heads, cols, rows]: a column's rows side by side); the matrix
// memory keeps n [heads, rows] and m [heads] behind all heads' S.  Memory is
// never cleared: a sequence whose first token of the step sits at position 0 starts from zeros (m from 0)
// whatever its slot holds.  Gates, decays, their logarithms and exponentials, n, m and S are float whatever T is;
// the gates' pre-activations come in as float.
//
// The decomposition is the one of the other recurrences of this package: a block owns one (sequence, head) and
// a slice of the columns and walks the sequence's tokens in order.  A column is shared by LPC neighbouring
// lanes, each holding RT consecutive rows of it in registers; a sum over the rows ends with log2(LPC) shuffles.
// Tokens are taken TC at a time through shared memory (coalesced loads, converted to float once; the next TC
// tokens' loads are in flight, in registers, while the steps run).  For the matrix memory the first column group
// of every warp carries n instead of a column of S (the same recurrence with v = 1), so that n . q is one
// shuffle away and no step needs a barrier; the first warp works out the gates of the TC tokens, each lane
// walking m from the value the block carries, in token order, so that m never depends on where a portion was cut.
#include "common.cuh"

using namespace vapi;

constexpr int LM_THREADS = 128;
constexpr int LM_MLSTM = 0, LM_GLA = 1;
constexpr int LM_GROUP = 4;                                   // tokens whose sums over the rows are taken together

__device__ __forceinline__ float lm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <int LPC>
__device__ __forceinline__ float lm_lanes_sum(float v) {
#pragma unroll
    for (int o = LPC >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// CH consecutive elements of a row vector as one thread brings them: with 16-byte loads where the addresses allow
template <int BYTES> struct LmRaw;
template <> struct __align__(8) LmRaw<8> { uint2 x; };
template <> struct __align__(16) LmRaw<16> { uint4 x; };
template <> struct __align__(16) LmRaw<32> { uint4 x, y; };
template <typename T, int CH>
union LmPiece {
    LmRaw<CH * (int)sizeof(T)> raw;
    T v[CH];
    __device__ LmPiece() {}
};

template <typename T, int RT, int LPC, int MODE>
struct LmShape {
    static constexpr int RP = RT * LPC;                        // rows, padded to what the lanes hold
    static constexpr int LANE = RT + 4;                        // floats from one lane's rows to the next lane's
    static constexpr int RPP = LANE * LPC;                     // a row vector in shared memory
    static constexpr int TC = RP > 128 ? 8 : 16;               // tokens a round
    static constexpr int G = 32 / LPC;                         // column groups a warp
    static constexpr int WARPS = LM_THREADS / 32;
    static constexpr int CW = MODE == LM_MLSTM ? G - 1 : G;    // columns of S a warp
    static constexpr int CB = CW * WARPS;                      // columns of S a block
    static constexpr int NV = MODE == LM_GLA ? 3 : 2;          // row vectors a token: k, q (, decay)
    static constexpr int NPT = TC * RP / LM_THREADS;           // row elements per thread and vector
    static constexpr int CH = NPT >= 8 ? 8 : 4;                // of which so many lie side by side in one token's row
    static constexpr int NCH = NPT / CH;
    static constexpr int VPT = (TC * CB + LM_THREADS - 1) / LM_THREADS;
    static_assert(RT % 4 == 0 && (TC * RP) % LM_THREADS == 0, "rows per lane come in fours");
    static_assert(NPT % CH == 0 && RT % CH == 0, "a thread's piece lies within one lane's rows");
    static __device__ __forceinline__ int pad(int r) { return r + (r / RT) * 4; }
};

template <typename T, int RT, int LPC, int MODE>
__global__ void __launch_bounds__(LM_THREADS)
linear_memory_kernel(const T* __restrict__ qkv, long long qkv_stride, int q_off, int k_off, int v_off,
                     const float* __restrict__ gates, long long gates_stride, const float* __restrict__ gate_bias,
                     float gate_param, float q_scale, float floor_eps, float* __restrict__ state, long long slot_stride,
                     const int* __restrict__ state_slots, const int* __restrict__ cu_q, const int* __restrict__ positions,
                     float* __restrict__ out, int nh, int rows, int cols, int num_slots, int wide_loads, int gates_are_decays,
                     int* __restrict__ status) {
    using Sh = LmShape<T, RT, LPC, MODE>;
    constexpr int TC = Sh::TC, RPP = Sh::RPP, RP = Sh::RP, CB = Sh::CB, VPT = Sh::VPT, CH = Sh::CH, NCH = Sh::NCH;
    __shared__ __align__(16) float sk[TC * RPP], sq[TC * RPP];
    __shared__ __align__(16) float sa[MODE == LM_GLA ? TC * RPP : 4];
    __shared__ float sv[TC * CB];
    __shared__ float s_keep[TC], s_take[TC], s_floor[TC], s_li[TC], s_lf[TC];
    const int s = blockIdx.z, h = blockIdx.y;
    const int col0 = blockIdx.x * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane / LPC, sl = lane % LPC;
    const bool is_n = MODE == LM_MLSTM && grp == 0;
    const int lc = MODE == LM_MLSTM ? warp * Sh::CW + grp - 1 : warp * Sh::CW + grp;     // column within the block
    const int col = col0 + lc;
    const bool col_ok = !is_n && col < cols;
    const int r0 = sl * RT;
    const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
    if (qlen <= 0) return;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0 && status) atomicExch(status, 3);
        return;
    }
    float* S_glob = state + (size_t)slot * slot_stride + ((size_t)h * rows) * cols;
    float* n_glob = state + (size_t)slot * slot_stride + (size_t)nh * rows * cols + (size_t)h * rows;
    float* m_glob = state + (size_t)slot * slot_stride + (size_t)nh * rows * cols + (size_t)nh * rows + h;
    const float bias_i = (MODE == LM_MLSTM && gate_bias) ? gate_bias[h] : 0.f;
    const float bias_f = (MODE == LM_MLSTM && gate_bias) ? gate_bias[nh + h] : 0.f;
    pdl_wait();
    // the state is asked for before it is known whether the sequence starts here, so that a decode step's loads
    // (the slot's state and the position) are in flight together; a fresh sequence drops what came
    // (a column's rows lie side by side in the slot, so a lane's rows are one run of floats and a warp's loads whole lines)
    float S[RT];
    float* S_mine = is_n ? n_glob + r0 : S_glob + (size_t)(col_ok ? col : 0) * rows + r0;
    const bool mine = is_n || col_ok;
    if (wide_loads & 2) {
#pragma unroll
        for (int j = 0; j < RT; j += 4) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mine && r0 + j < rows) x = *reinterpret_cast<const float4*>(S_mine + j);       // (rows come in fours)
            S[j] = x.x, S[j + 1] = x.y, S[j + 2] = x.z, S[j + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < RT; ++j) S[j] = (mine && r0 + j < rows) ? S_mine[j] : 0.f;
    }
    float m_run = MODE == LM_MLSTM ? *m_glob : 0.f;                      // (every lane of the first warp carries it)
    const bool fresh = positions[t0] == 0;
    if (fresh) {
        m_run = 0.f;
#pragma unroll
        for (int j = 0; j < RT; ++j) S[j] = 0.f;
    }

    // the next round's inputs, in registers: a thread brings pieces of CH neighbouring rows of one token (piece j
    // starts at element (threadIdx.x + j * LM_THREADS) * CH of the round's [TC, RP] rows)
    LmPiece<T, CH> ra[NCH], rb[NCH];
    LmPiece<float, CH> rz[MODE == LM_GLA ? NCH : 1];
    T rv[VPT];
    float g_i = 0.f, g_f = 0.f;
    auto fetch = [&](int first) {
        const int count = min(TC, qlen - first);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int idx = (threadIdx.x + j * LM_THREADS) * CH;
            const int tt = idx / RP, r = idx - tt * RP;
            const T* row = qkv + (size_t)(t0 + first + tt) * qkv_stride + h * rows + r;
            const float* zrow = gates + (size_t)(t0 + first + tt) * gates_stride + h * rows + r;
            if ((wide_loads & 1) && tt < count && r < rows) {          // (rows is a multiple of CH then: the piece is whole)
                ra[j].raw = *reinterpret_cast<const LmRaw<CH * (int)sizeof(T)>*>(row + k_off);
                rb[j].raw = *reinterpret_cast<const LmRaw<CH * (int)sizeof(T)>*>(row + q_off);
                if (MODE == LM_GLA) rz[j].raw = *reinterpret_cast<const LmRaw<CH * 4>*>(zrow);
            } else {
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const bool ok = tt < count && r + i < rows;
                    ra[j].v[i] = ok ? row[k_off + i] : from_f32<T>(0.f);
                    rb[j].v[i] = ok ? row[q_off + i] : from_f32<T>(0.f);
                    if (MODE == LM_GLA) rz[j].v[i] = ok ? zrow[i] : 0.f;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < VPT; ++e) {
            const int idx = threadIdx.x + e * LM_THREADS;
            const int tt = idx / CB, c = idx - tt * CB;
            const bool ok = idx < TC * CB && tt < count && col0 + c < cols;
            rv[e] = ok ? qkv[(size_t)(t0 + first + tt) * qkv_stride + v_off + h * cols + col0 + c] : from_f32<T>(0.f);
        }
        if (MODE == LM_MLSTM && (int)threadIdx.x < count) {
            g_i = gates[(size_t)(t0 + first + threadIdx.x) * gates_stride + h];
            g_f = gates[(size_t)(t0 + first + threadIdx.x) * gates_stride + nh + h];
        }
    };
    fetch(0);
    for (int first = 0; first < qlen; first += TC) {
        const int count = min(TC, qlen - first);
        __syncthreads();                                    // the steps of the last round have read shared memory
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int idx = (threadIdx.x + j * LM_THREADS) * CH;
            const int tt = idx / RP, r = idx - tt * RP;
            float4* dk = reinterpret_cast<float4*>(sk + tt * RPP + Sh::pad(r));
            float4* dq = reinterpret_cast<float4*>(sq + tt * RPP + Sh::pad(r));
            float4* da = reinterpret_cast<float4*>(sa + (MODE == LM_GLA ? tt * RPP + Sh::pad(r) : 0));
#pragma unroll
            for (int i = 0; i < CH; i += 4) {
                dk[i / 4] = make_float4(to_f32(ra[j].v[i]), to_f32(ra[j].v[i + 1]), to_f32(ra[j].v[i + 2]), to_f32(ra[j].v[i + 3]));
                dq[i / 4] = make_float4(to_f32(rb[j].v[i]) * q_scale, to_f32(rb[j].v[i + 1]) * q_scale,
                                        to_f32(rb[j].v[i + 2]) * q_scale, to_f32(rb[j].v[i + 3]) * q_scale);
                if (MODE == LM_GLA) {
                    float4 a = make_float4(rz[j].v[i], rz[j].v[i + 1], rz[j].v[i + 2], rz[j].v[i + 3]);
                    if (!gates_are_decays) {
                        a.x = expf(lm_logsigmoid(a.x) * gate_param);
                        a.y = expf(lm_logsigmoid(a.y) * gate_param);
                        a.z = expf(lm_logsigmoid(a.z) * gate_param);
                        a.w = expf(lm_logsigmoid(a.w) * gate_param);
                    }
                    da[i / 4] = a;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < VPT; ++e)
            if (threadIdx.x + e * LM_THREADS < TC * CB) sv[threadIdx.x + e * LM_THREADS] = to_f32(rv[e]);
        if (MODE == LM_MLSTM && warp == 0) {
            if (lane < count) {
                s_li[lane] = gate_param * tanhf((g_i + bias_i) / gate_param);
                s_lf[lane] = lm_logsigmoid(gate_param * tanhf((g_f + bias_f) / gate_param));
            }
            __syncwarp();
            // lane t walks m over the round's tokens 0 .. t, as the recurrence does, and keeps its own token's factors
            float m = m_run, m_before = m_run;
            for (int u = 0; u <= min(lane, count - 1); ++u) {
                m_before = m;
                m = fmaxf(s_lf[u] + m, s_li[u]);
            }
            if (lane < count) {
                s_keep[lane] = expf(s_lf[lane] + m_before - m);
                s_take[lane] = expf(s_li[lane] - m);
                s_floor[lane] = expf(-m);
            }
            m_run = __shfl_sync(0xffffffffu, m, count - 1);
        }
        __syncthreads();
        if (first + TC < qlen) fetch(first + TC);           // in flight while these steps run
        // four tokens at a time: their updates follow one another, their sums over the rows travel together, so
        // that one token's shuffles are in flight beside the next one's arithmetic
        for (int g0 = 0; g0 < count; g0 += LM_GROUP) {
            float part[LM_GROUP];
#pragma unroll
            for (int u = 0; u < LM_GROUP; ++u) {
                const int tt = g0 + u;
                part[u] = 0.f;
                if (tt >= count) continue;                  // (the same for the whole block)
                const float4* k4 = reinterpret_cast<const float4*>(sk + tt * RPP + sl * Sh::LANE);
                const float4* q4 = reinterpret_cast<const float4*>(sq + tt * RPP + sl * Sh::LANE);
                const float4* a4 = reinterpret_cast<const float4*>(sa + (MODE == LM_GLA ? tt * RPP + sl * Sh::LANE : 0));
                const float vv = is_n ? 1.f : sv[tt * CB + (lc < CB ? lc : 0)];
                float dot0 = 0.f, dot1 = 0.f;
                if (MODE == LM_MLSTM) {
                    const float keep = s_keep[tt], tv = s_take[tt] * vv;
#pragma unroll
                    for (int r4 = 0; r4 < RT / 4; ++r4) {
                        const float4 kv = k4[r4], qv = q4[r4];
                        S[4 * r4] = fmaf(kv.x, tv, keep * S[4 * r4]);
                        S[4 * r4 + 1] = fmaf(kv.y, tv, keep * S[4 * r4 + 1]);
                        S[4 * r4 + 2] = fmaf(kv.z, tv, keep * S[4 * r4 + 2]);
                        S[4 * r4 + 3] = fmaf(kv.w, tv, keep * S[4 * r4 + 3]);
                        dot0 = fmaf(S[4 * r4], qv.x, dot0);
                        dot1 = fmaf(S[4 * r4 + 1], qv.y, dot1);
                        dot0 = fmaf(S[4 * r4 + 2], qv.z, dot0);
                        dot1 = fmaf(S[4 * r4 + 3], qv.w, dot1);
                    }
                } else {
#pragma unroll
                    for (int r4 = 0; r4 < RT / 4; ++r4) {
                        const float4 kv = k4[r4], qv = q4[r4], av = a4[r4];
                        S[4 * r4] = fmaf(kv.x, vv, av.x * S[4 * r4]);
                        S[4 * r4 + 1] = fmaf(kv.y, vv, av.y * S[4 * r4 + 1]);
                        S[4 * r4 + 2] = fmaf(kv.z, vv, av.z * S[4 * r4 + 2]);
                        S[4 * r4 + 3] = fmaf(kv.w, vv, av.w * S[4 * r4 + 3]);
                        dot0 = fmaf(S[4 * r4], qv.x, dot0);
                        dot1 = fmaf(S[4 * r4 + 1], qv.y, dot1);
                        dot0 = fmaf(S[4 * r4 + 2], qv.z, dot0);
                        dot1 = fmaf(S[4 * r4 + 3], qv.w, dot1);
                    }
                }
                part[u] = dot0 + dot1;
            }
#pragma unroll
            for (int o = LPC >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < LM_GROUP; ++u) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
            }
            if (MODE == LM_MLSTM) {
#pragma unroll
                for (int u = 0; u < LM_GROUP; ++u) {
                    const float nq = __shfl_sync(0xffffffffu, part[u], 0);    // the first group's sum is n . q
                    part[u] = part[u] / (fmaxf(fabsf(nq), s_floor[min(g0 + u, TC - 1)]) + floor_eps);
                }
            }
            if (sl == 0 && col_ok) {
#pragma unroll
                for (int u = 0; u < LM_GROUP; ++u)
                    if (g0 + u < count) out[((size_t)(t0 + first + g0 + u) * nh + h) * cols + col] = part[u];
            }
        }
    }
    pdl_trigger();                                          // (the next kernel is let go when the walk is over)
    const bool put = is_n ? (blockIdx.x == 0 && warp == 0) : col_ok;
    if (wide_loads & 2) {
#pragma unroll
        for (int j = 0; j < RT; j += 4)
            if (put && r0 + j < rows) *reinterpret_cast<float4*>(S_mine + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < RT; ++j)
            if (put && r0 + j < rows) S_mine[j] = S[j];
    }
    if (MODE == LM_MLSTM && blockIdx.x == 0 && threadIdx.x == 0) *m_glob = m_run;
}

// alpha = sigmoid(z)^p = exp(p logsigmoid(z)) over [n, width] rows, in place: once per element for a step with long
// portions, where every block of a head would otherwise work out the head's decays again
__global__ void __launch_bounds__(256)
decay_from_logits_kernel(float* __restrict__ z, long long stride, int width, long long total, float p) {
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float* e = z + (i / width) * stride + (i % width);
        *e = expf(lm_logsigmoid(*e) * p);
    }
    pdl_trigger();
}

// (RT, LPC) by the number of rows: 8 x 4 up to 32, 8 x 8 up to 64, 16 x 8 up to 128, 16 x 16 up to 256.  A state of
// 65 to 128 rows takes 8 x 16 instead while the grid would leave schedulers without a warp (`fine`): twice the
// threads share a column and a token's chain of updates is half as long.  (The matrix memory gives a column group of
// every warp to n, so its finer split spends half of its lanes there; with one prompt in the step that still
// beats one warp a scheduler walking twice the rows.)
#define LM_DISPATCH(ROWS, FINE, CALL)                               \
    do {                                                            \
        if ((ROWS) <= 32) { CALL(8, 4); }                           \
        else if ((ROWS) <= 64) { CALL(8, 8); }                      \
        else if ((ROWS) <= 128 && (FINE)) { CALL(8, 16); }          \
        else if ((ROWS) <= 128) { CALL(16, 8); }                    \
        else { CALL(16, 16); }                                      \
    } while (0)

static inline int lm_lpc(int rows, bool fine) { return rows <= 32 ? 4 : (rows <= 64 ? 8 : (rows <= 128 ? (fine ? 16 : 8) : 16)); }

static int lm_launch(int mode, const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off, int dtype,
                     float* gates, long long gates_stride, const float* gate_bias, float gate_param, float q_scale,
                     float floor_eps, float* state, long long slot_stride, const int* state_slots, const int* cu_q,
                     const int* positions, float* out, int total_rows, int num_seqs, int nh, int rows, int cols, int num_slots,
                     int max_q, int* status, cudaStream_t stream, const char* what) {
    if (num_seqs <= 0) return 0;
    if (nh <= 0 || rows <= 0 || rows > 256 || cols <= 0)
        return fail(-1, "%s: %d heads, state %d x %d (rows up to 256)", what, nh, rows, cols);
    if (dtype != VAPI_F32 && dtype != VAPI_BF16) return fail(-2, "%s: unsupported dtype %d", what, dtype);
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int g_wide = 32 / lm_lpc(rows, false);                               // column groups a warp of the ordinary split
    const int wide = (mode == LM_MLSTM ? g_wide - 1 : g_wide) * (LM_THREADS / 32);
    const bool fine = rows > 64 && rows <= 128 && (long long)((cols + wide - 1) / wide) * nh * num_seqs < 2LL * sms;
    const int g = 32 / lm_lpc(rows, fine);
    const int cb = (mode == LM_MLSTM ? g - 1 : g) * (LM_THREADS / 32);
    dim3 grid((cols + cb - 1) / cb, nh, num_seqs);
    if (grid.y > 65535 || grid.z > 65535) return fail(-1, "%s: %d heads x %d sequences are too many", what, nh, num_seqs);
    const bool early = max_q < 16;                         // decode steps may start beside the kernel before; long walks may not
    cudaError_t e = cudaSuccess;
    // 16-byte loads of the row vectors: every piece of 8 (4 up to 32 rows) starts on its boundary
    const int ch = rows <= 32 ? 4 : 8;
    const size_t esz = dtype == VAPI_F32 ? 4 : 2;
    int wide_loads = rows % ch == 0 && q_off % ch == 0 && k_off % ch == 0 && qkv_stride % ch == 0 &&
                     (size_t)qkv % (ch * esz > 16 ? 16 : ch * esz) == 0;
    if (mode == LM_GLA) wide_loads = wide_loads && gates_stride % ch == 0 && (size_t)gates % 16 == 0;
    // 16-byte accesses of the state: a lane's run of rows starts on a boundary (n and m lie behind whole columns)
    if (rows % 4 == 0 && slot_stride % 4 == 0 && (size_t)state % 16 == 0) wide_loads |= 2;
    int gates_are_decays = 0;
    if (mode == LM_GLA && !early) {
        const long long total = (long long)total_rows * nh * rows;
        const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
        e = launch_if(false, decay_from_logits_kernel, dim3(blocks > 0 ? blocks : 1), 256, 0, stream, gates, gates_stride,
                      nh * rows, total, gate_param);
        if (e != cudaSuccess) return check_launch(what, e);
        gates_are_decays = 1;
    }
#define LM_CALL_MODE(RT, LPC, M)                                                                                           \
    if (dtype == VAPI_F32)                                                                                                 \
        e = launch_if(early, linear_memory_kernel<float, RT, LPC, M>, grid, LM_THREADS, 0, stream, (const float*)qkv,      \
                      qkv_stride, q_off, k_off, v_off, gates, gates_stride, gate_bias, gate_param, q_scale, floor_eps,     \
                      state, slot_stride, state_slots, cu_q, positions, out, nh, rows, cols, num_slots, wide_loads,        \
                      gates_are_decays, status);                                                                           \
    else                                                                                                                   \
        e = launch_if(early, linear_memory_kernel<__nv_bfloat16, RT, LPC, M>, grid, LM_THREADS, 0, stream,                 \
                      (const __nv_bfloat16*)qkv, qkv_stride, q_off, k_off, v_off, gates, gates_stride, gate_bias,          \
                      gate_param, q_scale, floor_eps, state, slot_stride, state_slots, cu_q, positions, out, nh, rows,     \
                      cols, num_slots, wide_loads, gates_are_decays, status)
#define LM_CALL_A(RT, LPC) LM_CALL_MODE(RT, LPC, LM_MLSTM)
#define LM_CALL_B(RT, LPC) LM_CALL_MODE(RT, LPC, LM_GLA)
    if (mode == LM_MLSTM) LM_DISPATCH(rows, fine, LM_CALL_A);
    else LM_DISPATCH(rows, fine, LM_CALL_B);
#undef LM_CALL_A
#undef LM_CALL_B
#undef LM_CALL_MODE
    return check_launch(what, e);
}

// qkv [n, *]: q heads [nh, rows] at q_off, k heads [nh, rows] at k_off, v heads [nh, cols] at v_off of a row of
// `qkv_stride` elements.  gates [n, *] float: the input gates' pre-activations [nh], then the forget gates' [nh];
// gate_bias [2 * nh] likewise (may be null).  state: S [nh, cols, rows] (column by column), n [nh, rows], m [nh] per slot.  out [n, nh * cols] float.
VAPI_EXPORT int vapi_matrix_memory(const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off, int dtype,
                                   const float* gates, long long gates_stride, const float* gate_bias, float cap,
                                   float q_scale, float floor_eps, float* state, long long slot_stride,
                                   const int* state_slots, const int* cu_q, const int* positions, float* out, int num_seqs,
                                   int nh, int rows, int cols, int num_slots, int max_q, int* status, cudaStream_t stream) {
    if (!(cap > 0.f)) return fail(-1, "matrix_memory: the gates' cap must be positive");
    return lm_launch(LM_MLSTM, qkv, qkv_stride, q_off, k_off, v_off, dtype, const_cast<float*>(gates), gates_stride, gate_bias,
                     cap, q_scale, floor_eps, state, slot_stride, state_slots, cu_q, positions, out, 0, num_seqs, nh, rows, cols,
                     num_slots, max_q, status, stream, "matrix_memory");
}

// As above without gates' scalars: decay_logits [num_tokens, *] float holds z [nh, rows] per token; alpha = sigmoid(z)^inv_tau.
// A step with portions of 16 tokens or more turns z into alpha in place first (decay_logits is scratch then).
// state: S [nh, cols, rows] (column by column) per slot.
VAPI_EXPORT int vapi_gated_linear_attention(const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off, int dtype,
                                            float* decay_logits, long long decay_stride, float inv_tau, float q_scale,
                                            float* state, long long slot_stride, const int* state_slots, const int* cu_q,
                                            const int* positions, float* out, int num_tokens, int num_seqs, int nh, int rows,
                                            int cols, int num_slots, int max_q, int* status, cudaStream_t stream) {
    return lm_launch(LM_GLA, qkv, qkv_stride, q_off, k_off, v_off, dtype, decay_logits, decay_stride, nullptr, inv_tau,
                     q_scale, 0.f, state, slot_stride, state_slots, cu_q, positions, out, num_tokens, num_seqs, nh, rows, cols,
                     num_slots, max_q, status, stream, "gated_linear_attention");
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
