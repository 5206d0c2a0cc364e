// Gated linear attention: a recurrent mixer with a matrix of state per head.
//
//   a_t  = sigmoid(z_t + b)^(1/tau)                           one decay per key channel (z_t: a projection of the input)
//   S_t  = diag(a_t) S_{t-1} + k_t v_t^T                      S: [d, dv] float per head and sequence (stored [dv, d]: a
//                                                             lane's run of key channels of one column is contiguous)
//   o_t  = S_t^T (q_t * q_scale)
//
// followed, in a second kernel, by an RMS norm of each head's o over dv, a gate silu(g) and the rounding to the
// activation type.  Decays, their logarithms, the state and o are float whatever the projections are stored in.
// The state lives in the cache (one [H, d, dv] block per slot and line): a step loads it, runs its tokens in
// order and writes it back, so a prompt, a prompt that continues and a decode step are the same launch.
#include "common.cuh"

#include <math_constants.h>
#include <type_traits>

namespace janis {

constexpr int GLA_KS = 16;         // lanes that share a column of the state (each holds a run of DPT key channels)
constexpr int GLA_COLS = 8;        // value columns per CTA

struct GlaRows {
    int row_elems;                 // elements per row of the projected step
    int q_off, k_off, v_off;       // where q [H, d], k [H, d] and v [H, dv] start in a row
    int H, d, dv;
    float q_scale, inv_tau;
};

__device__ __forceinline__ float log_sigmoid(float z) {       // -softplus(-z), stable at both ends
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// a[t, c] = sigmoid(z[t, c] + b[c])^(1/tau) as floats, once per step (every column group of a head reads them)
template <typename T>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const T* __restrict__ z, const T* __restrict__ bias, float* __restrict__ a, size_t n, int width, float inv_tau) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        a[i] = expf(log_sigmoid(to_float(z[i]) + to_float(bias[i % width])) * inv_tau);
}

// grid (sequences, heads, ceil(dv / GLA_COLS)); 128 threads: thread = (column, ks), ks fastest, so that the 16
// lanes of a column sit in one half of a warp (tiles of 16 tokens, or of 8 at the largest key sizes).  Lane ks holds key channels ks * DPT .. ks * DPT + DPT - 1 of its
// column (DPT a multiple of 4, 16 * DPT >= d; channels beyond d hold zeros and decay 1).  A token's q, k and
// decays lie in shared memory as runs of DPT floats, each followed by 4 floats of padding, so that the lanes'
// 16-byte reads fall into different banks.
template <typename T, int DPT>
__global__ void __launch_bounds__(GLA_COLS * GLA_KS)
gla_scan_kernel(const T* __restrict__ rows, GlaRows g, const float* __restrict__ decay,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                const int* __restrict__ seq_start, const int* __restrict__ seq_end, float* __restrict__ state,
                float* __restrict__ o_out) {
    constexpr int RUN = DPT + 4, TOK = GLA_KS * RUN;       // floats of a lane's run, of a token
    constexpr int GLA_TT = DPT >= 16 ? 8 : 16;             // tokens staged per round (static shared memory stays under 48 KB)
    __shared__ __align__(16) float q_s[GLA_TT * TOK];
    __shared__ __align__(16) float k_s[GLA_TT * TOK];
    __shared__ __align__(16) float a_s[GLA_TT * TOK];
    __shared__ float v_s[GLA_TT * GLA_COLS];
    const int d = g.d, dv = g.dv, H = g.H;
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int tid = threadIdx.x, ks = tid % GLA_KS, col = col0 + tid / GLA_KS;
    const bool live = col < dv;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    grid_dependency_wait();
    float S[DPT];
    float* st = slot >= 0 ? state + ((size_t)slot * H + h) * d * dv : nullptr;
#pragma unroll
    for (int ii = 0; ii < DPT; ++ii) {
        const int i = ks * DPT + ii;
        S[ii] = (st != nullptr && live && i < d) ? st[(size_t)col * d + i] : 0.f;
    }
    // A tile's q, k and decays travel through registers: a fixed number of elements a thread, all of their loads
    // asked for at once, and those of the next tile while this one is computed.  Tokens beyond the sequence's end
    // become q = k = v = 0 and decay 1, which change nothing, so a tile always runs all of its tokens.
    constexpr int NT = GLA_COLS * GLA_KS, WIDTH = GLA_KS * DPT;
    constexpr int PER = GLA_TT * WIDTH / NT;               // elements of each of q, k and the decays a thread carries
    constexpr int CH = WIDTH / 8;                          // pieces of 8 channels a token
    float qv[PER], kv[PER], av[PER], vv = 0.f;
    // 16-byte loads (8 channels of one token a piece) where the rows allow it, else element by element (also at the
    // smallest key sizes, where the pieces' places in shared memory would fall into few banks)
    const bool vec = DPT >= 8 && d % 8 == 0 && g.row_elems % 8 == 0 && g.q_off % 8 == 0 && g.k_off % 8 == 0 &&
                     (((uintptr_t)rows | (uintptr_t)decay) & 15) == 0 && sizeof(T) == 2;
    auto fetch = [&](int t0) {
        if (vec) {
#pragma unroll
            for (int e = 0; e < PER / 8; ++e) {
                const int u = tid + e * NT, tt = u / CH, c0 = (u % CH) * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    qv[e * 8 + j] = kv[e * 8 + j] = 0.f;
                    av[e * 8 + j] = 1.f;
                }
                if (t0 + tt < n_tok && c0 < d) {
                    const T* row = rows + (size_t)(row0 + t0 + tt) * g.row_elems;
                    Vec16<T>::load(row + g.q_off + h * d + c0, &qv[e * 8]);      // (Vec16<bf16>: 8 values; this path is bfloat16 only)
                    Vec16<T>::load(row + g.k_off + h * d + c0, &kv[e * 8]);
                    const float4* dp = reinterpret_cast<const float4*>(decay + (size_t)(row0 + t0 + tt) * H * d + h * d + c0);
                    const float4 d0 = dp[0], d1 = dp[1];
                    av[e * 8 + 0] = d0.x; av[e * 8 + 1] = d0.y; av[e * 8 + 2] = d0.z; av[e * 8 + 3] = d0.w;
                    av[e * 8 + 4] = d1.x; av[e * 8 + 5] = d1.y; av[e * 8 + 6] = d1.z; av[e * 8 + 7] = d1.w;
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int u = tid + e * NT;
                const int tt = u / WIDTH, c = u % WIDTH;
                qv[e] = kv[e] = 0.f;
                av[e] = 1.f;
                if (t0 + tt < n_tok && c < d) {
                    const T* row = rows + (size_t)(row0 + t0 + tt) * g.row_elems;
                    qv[e] = to_float(row[g.q_off + h * d + c]);
                    kv[e] = to_float(row[g.k_off + h * d + c]);
                    av[e] = decay[(size_t)(row0 + t0 + tt) * H * d + h * d + c];
                }
            }
        }
        vv = 0.f;
        if (tid < GLA_TT * GLA_COLS) {
            const int tt = tid / GLA_COLS, c = col0 + tid % GLA_COLS;
            if (t0 + tt < n_tok && c < dv) vv = to_float(rows[(size_t)(row0 + t0 + tt) * g.row_elems + g.v_off + h * dv + c]);
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < n_tok; t0 += GLA_TT) {
        __syncthreads();                       // the tile before has been read
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            int tt, c;
            if (vec) {
                const int u = tid + (e / 8) * NT;
                tt = u / CH;
                c = (u % CH) * 8 + e % 8;
            } else {
                const int u = tid + e * NT;
                tt = u / WIDTH;
                c = u % WIDTH;
            }
            const int at = tt * TOK + (c / DPT) * RUN + c % DPT;
            q_s[at] = qv[e] * g.q_scale;
            k_s[at] = kv[e];
            a_s[at] = av[e];
        }
        if (tid < GLA_TT * GLA_COLS) v_s[tid] = vv;
        __syncthreads();
        if (t0 + GLA_TT < n_tok) fetch(t0 + GLA_TT);
        // the tile's tokens in order; each lane's share of o_t stays in a register until the tile is done
        float part_o[GLA_TT];
        const int tt_n = min(GLA_TT, n_tok - t0);
        // a whole tile runs without a test per token (its reads may then be asked for tokens ahead); the last tile of
        // a prompt, and the single token of a decode step, skip the tokens that are not there
        auto run_tokens = [&](auto guarded) {
#pragma unroll
            for (int tt = 0; tt < GLA_TT; ++tt) {
                part_o[tt] = 0.f;
                if (decltype(guarded)::value && tt >= tt_n) continue;
                const float v = v_s[tt * GLA_COLS + tid / GLA_KS];
                const float4* qq = reinterpret_cast<const float4*>(q_s + tt * TOK + ks * RUN);
                const float4* kk = reinterpret_cast<const float4*>(k_s + tt * TOK + ks * RUN);
                const float4* aa = reinterpret_cast<const float4*>(a_s + tt * TOK + ks * RUN);
                float part[4] = {0.f, 0.f, 0.f, 0.f};           // four chains, added in a fixed order
#pragma unroll
                for (int i4 = 0; i4 < DPT / 4; ++i4) {
                    const float4 q4 = qq[i4], k4 = kk[i4], a4 = aa[i4];
                    S[4 * i4 + 0] = fmaf(a4.x, S[4 * i4 + 0], k4.x * v);
                    S[4 * i4 + 1] = fmaf(a4.y, S[4 * i4 + 1], k4.y * v);
                    S[4 * i4 + 2] = fmaf(a4.z, S[4 * i4 + 2], k4.z * v);
                    S[4 * i4 + 3] = fmaf(a4.w, S[4 * i4 + 3], k4.w * v);
                    part[0] = fmaf(S[4 * i4 + 0], q4.x, part[0]);
                    part[1] = fmaf(S[4 * i4 + 1], q4.y, part[1]);
                    part[2] = fmaf(S[4 * i4 + 2], q4.z, part[2]);
                    part[3] = fmaf(S[4 * i4 + 3], q4.w, part[3]);
                }
                part_o[tt] = (part[0] + part[1]) + (part[2] + part[3]);
            }
        };
        if (tt_n == GLA_TT) run_tokens(std::false_type{});
        else run_tokens(std::true_type{});
        // the 16 lanes of a column add their shares of all the tile's tokens at once: every stage halves the tokens
        // a lane still carries (the lanes whose bit is set keep the upper half), so 15 shuffles do what 64 would
        int n = GLA_TT;
#pragma unroll
        for (int off = GLA_KS / 2; off >= 1; off >>= 1) {
            const bool upper = (ks & off) != 0;
            if (n > 1) {
                const int half = n / 2;
#pragma unroll
                for (int i = 0; i < GLA_TT / 2; ++i)
                    if (i < half) {
                        const float mine = upper ? part_o[i + half] : part_o[i];
                        const float theirs = upper ? part_o[i] : part_o[i + half];
                        part_o[i] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
                    }
                n = half;
            } else {
                part_o[0] += __shfl_xor_sync(0xffffffffu, part_o[0], off);
            }
        }
        // lane ks now holds token ks * GLA_TT / 16 of the tile (lanes that share a token hold the same sum)
        constexpr int SHARE = GLA_KS / GLA_TT;              // 1, or 2 with tiles of 8 tokens
        const int tt = ks / SHARE;
        if (live && ks % SHARE == 0 && t0 + tt < n_tok) o_out[(size_t)(row0 + t0 + tt) * H * dv + h * dv + col] = part_o[0];
    }
    if (st != nullptr && live) {
#pragma unroll
        for (int ii = 0; ii < DPT; ++ii) {
            const int i = ks * DPT + ii;
            if (i < d) st[(size_t)col * d + i] = S[ii];
        }
    }
}

// ---------------------------------------------------------------------------
// Matrix memory with exponential gates (mLSTM): per head and sequence a matrix C [d, dv], a vector n [d] and a
// running maximum m, all float:
//
//   i_t = cap tanh((zi_t + bi) / cap),   f_t = logsigmoid(cap tanh((zf_t + bf) / cap))       (zi, zf: float logits)
//   m_t = max(f_t + m_{t-1}, i_t)                                                               (m starts at 0)
//   C_t = e^(f_t + m_{t-1} - m_t) C_{t-1} + e^(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
//   o_t = C_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
//
// Two kernels.  `mlstm_gates`: a warp per (sequence, head) runs the chain of maxima over the step's tokens, 32 at a
// time, as a scan over the maps m -> max(a, b + m) (two such maps compose to one of the same form), and leaves per
// (token, head) the three factors keep = e^(f + m' - m), take = e^(i - m), floor = e^(-m); m is loaded from and
// written back to the cache.  `mlstm_scan`: the recurrence itself in the layout of the scan above (16 lanes a column
// of C, each holding a run of key channels), with n as one more column whose value is 1 in every CTA (so every
// CTA owns a copy of n: the cache keeps one per group of columns and no CTA waits for another).  A tile's n . q pass
// through shared memory and its results are divided and written while the next tile is staged.
// ---------------------------------------------------------------------------
template <int DUMMY>
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const float* __restrict__ z, const float* __restrict__ bias, float cap, int H,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_end, float* __restrict__ m_state,
                   float* __restrict__ coef) {
    const int seq = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    const float bi = bias[h], bf = bias[H + h];
    if (n_tok <= 0) return;
    grid_dependency_wait();
    float m = slot >= 0 ? m_state[(size_t)slot * H + h] : 0.f;
    for (int t0 = 0; t0 < n_tok; t0 += 32) {
        const bool in = t0 + lane < n_tok;
        float gi = -CUDART_INF_F, gf = 0.f;                  // beyond the end: the map that changes nothing
        if (in) {
            const float* zr = z + (size_t)(row0 + t0 + lane) * 2 * H;
            gi = cap * tanhf((zr[h] + bi) / cap);
            gf = log_sigmoid(cap * tanhf((zr[H + h] + bf) / cap));
        }
        float a = gi, b = gf;                                // the map m -> max(a, b + m) of this token, then of all up to it
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float pa = __shfl_up_sync(0xffffffffu, a, off), pb = __shfl_up_sync(0xffffffffu, b, off);
            if (lane >= off) {
                a = fmaxf(a, b + pa);
                b = b + pb;
            }
        }
        const float m_new = fmaxf(a, b + m);
        float m_prev = __shfl_up_sync(0xffffffffu, m_new, 1);
        if (lane == 0) m_prev = m;
        if (in) {
            float* c = coef + ((size_t)(row0 + t0 + lane) * H + h) * 3;
            c[0] = expf(gf + m_prev - m_new);
            c[1] = expf(gi - m_new);
            c[2] = expf(-m_new);
        }
        m = __shfl_sync(0xffffffffu, m_new, 31);
    }
    if (slot >= 0 && lane == 0) m_state[(size_t)slot * H + h] = m;
}

constexpr int MLSTM_GROUPS = GLA_COLS + 2;      // the value columns, the column of n, and one idle group that fills the last warp
constexpr int MLSTM_THREADS = MLSTM_GROUPS * GLA_KS;

// (a decode step is over in a few waves of CTAs, so what an SM holds at once counts: four CTAs at the smallest key
// size, three at the middle one)
template <typename T, int DPT>
__global__ void __launch_bounds__(MLSTM_THREADS, DPT <= 4 ? 4 : (DPT <= 8 ? 3 : 1))
mlstm_scan_kernel(const T* __restrict__ rows, GlaRows g, const float* __restrict__ coef,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_end, float* __restrict__ state_c,
                  float* __restrict__ state_n, float* __restrict__ o_out) {
    constexpr int RUN = DPT + 4, TOK = GLA_KS * RUN;       // floats of a lane's run, of a token
    constexpr int TT = DPT >= 16 ? 8 : 16;                 // tokens staged per round
    __shared__ __align__(16) float q_s[TT * TOK];
    __shared__ __align__(16) float k_s[TT * TOK];
    __shared__ float v_s[TT * GLA_COLS];
    __shared__ float keep_s[TT], take_s[TT];
    __shared__ float floor_s[2][TT], nq_s[2][TT];          // by the tile's parity: a tile's results leave while the next is staged
    const int d = g.d, dv = g.dv, H = g.H;
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GLA_COLS, n_groups = gridDim.z;
    const int tid = threadIdx.x, ks = tid % GLA_KS, grp = tid / GLA_KS, col = col0 + grp;
    const bool is_n = grp == GLA_COLS;                     // the column of n: its value is 1
    const bool live = (grp < GLA_COLS && col < dv) || is_n;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    grid_dependency_wait();
    float S[DPT];
    float* st = nullptr;
    if (slot >= 0 && live)
        st = is_n ? state_n + (((size_t)slot * H + h) * n_groups + blockIdx.z) * d
                  : state_c + (((size_t)slot * H + h) * dv + col) * d;
#pragma unroll
    for (int ii = 0; ii < DPT; ++ii) {
        const int i = ks * DPT + ii;
        S[ii] = (st != nullptr && i < d) ? st[i] : 0.f;
    }
    constexpr int NT = GLA_COLS * GLA_KS, WIDTH = GLA_KS * DPT;       // the first NT threads stage a tile
    constexpr int PER = TT * WIDTH / NT;
    constexpr int CH = WIDTH / 8;
    float qv[PER], kv[PER], vv = 0.f, cf_keep = 1.f, cf_take = 0.f, cf_floor = 1.f;
    const bool vec = DPT >= 8 && d % 8 == 0 && g.row_elems % 8 == 0 && g.q_off % 8 == 0 && g.k_off % 8 == 0 &&
                     (((uintptr_t)rows) & 15) == 0 && sizeof(T) == 2;
    auto fetch = [&](int t0) {
        if (tid < NT) {
            if (vec) {
#pragma unroll
                for (int e = 0; e < PER / 8; ++e) {
                    const int u = tid + e * NT, tt = u / CH, c0 = (u % CH) * 8;
#pragma unroll
                    for (int j = 0; j < 8; ++j) qv[e * 8 + j] = kv[e * 8 + j] = 0.f;
                    if (t0 + tt < n_tok && c0 < d) {
                        const T* row = rows + (size_t)(row0 + t0 + tt) * g.row_elems;
                        Vec16<T>::load(row + g.q_off + h * d + c0, &qv[e * 8]);
                        Vec16<T>::load(row + g.k_off + h * d + c0, &kv[e * 8]);
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < PER; ++e) {
                    const int u = tid + e * NT;
                    const int tt = u / WIDTH, c = u % WIDTH;
                    qv[e] = kv[e] = 0.f;
                    if (t0 + tt < n_tok && c < d) {
                        const T* row = rows + (size_t)(row0 + t0 + tt) * g.row_elems;
                        qv[e] = to_float(row[g.q_off + h * d + c]);
                        kv[e] = to_float(row[g.k_off + h * d + c]);
                    }
                }
            }
            vv = 0.f;
            if (tid < TT * GLA_COLS) {
                const int tt = tid / GLA_COLS, c = col0 + tid % GLA_COLS;
                if (t0 + tt < n_tok && c < dv) vv = to_float(rows[(size_t)(row0 + t0 + tt) * g.row_elems + g.v_off + h * dv + c]);
            }
        } else if (tid - NT < TT) {
            // the tile's factors, a token a thread: keep 1, take 0 and floor 1 beyond the sequence's end change nothing
            const int tt = tid - NT;
            cf_keep = 1.f; cf_take = 0.f; cf_floor = 1.f;
            if (t0 + tt < n_tok) {
                const float* c = coef + ((size_t)(row0 + t0 + tt) * H + h) * 3;
                cf_keep = c[0]; cf_take = c[1]; cf_floor = c[2];
            }
        }
    };
    constexpr int SHARE = GLA_KS / TT;                      // lanes that end up with the same token's sum: 1, or 2 with tiles of 8 tokens
    const int my_tt = ks / SHARE;
    const bool writer = live && !is_n && ks % SHARE == 0;
    float held = 0.f;                                       // this lane's numerator of the tile before
    auto write_out = [&](int t0, int par) {
        // o = C^T q / (max(|n . q|, e^(-m)) + 1e-6), with n . q from the group that carries n
        if (writer && t0 + my_tt < n_tok)
            o_out[(size_t)(row0 + t0 + my_tt) * H * dv + h * dv + col] = held / (fmaxf(fabsf(nq_s[par][my_tt]), floor_s[par][my_tt]) + 1e-6f);
    };
    fetch(0);
    int par = 0;
    for (int t0 = 0; t0 < n_tok; t0 += TT, par ^= 1) {
        __syncthreads();                       // the tile before has been read, and its n . q stand in shared memory
        if (t0 > 0) write_out(t0 - TT, par ^ 1);
        if (tid >= NT && tid - NT < TT) {
            keep_s[tid - NT] = cf_keep;
            take_s[tid - NT] = cf_take;
            floor_s[par][tid - NT] = cf_floor;
        }
        if (tid < NT) {
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                int tt, c;
                if (vec) {
                    const int u = tid + (e / 8) * NT;
                    tt = u / CH;
                    c = (u % CH) * 8 + e % 8;
                } else {
                    const int u = tid + e * NT;
                    tt = u / WIDTH;
                    c = u % WIDTH;
                }
                const int at = tt * TOK + (c / DPT) * RUN + c % DPT;
                q_s[at] = qv[e] * g.q_scale;
                k_s[at] = kv[e];
            }
            if (tid < TT * GLA_COLS) v_s[tid] = vv;
        }
        __syncthreads();
        if (t0 + TT < n_tok) fetch(t0 + TT);
        float part_o[TT];
        const int tt_n = min(TT, n_tok - t0);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            part_o[tt] = 0.f;
            if (tt >= tt_n) continue;
            const float v = (is_n ? 1.f : (grp < GLA_COLS ? v_s[tt * GLA_COLS + grp] : 0.f)) * take_s[tt];
            const float keep = keep_s[tt];
            const float4* qq = reinterpret_cast<const float4*>(q_s + tt * TOK + ks * RUN);
            const float4* kk = reinterpret_cast<const float4*>(k_s + tt * TOK + ks * RUN);
            float part[4] = {0.f, 0.f, 0.f, 0.f};           // four chains, added in a fixed order
#pragma unroll
            for (int i4 = 0; i4 < DPT / 4; ++i4) {
                const float4 q4 = qq[i4], k4 = kk[i4];
                S[4 * i4 + 0] = fmaf(keep, S[4 * i4 + 0], k4.x * v);
                S[4 * i4 + 1] = fmaf(keep, S[4 * i4 + 1], k4.y * v);
                S[4 * i4 + 2] = fmaf(keep, S[4 * i4 + 2], k4.z * v);
                S[4 * i4 + 3] = fmaf(keep, S[4 * i4 + 3], k4.w * v);
                part[0] = fmaf(S[4 * i4 + 0], q4.x, part[0]);
                part[1] = fmaf(S[4 * i4 + 1], q4.y, part[1]);
                part[2] = fmaf(S[4 * i4 + 2], q4.z, part[2]);
                part[3] = fmaf(S[4 * i4 + 3], q4.w, part[3]);
            }
            part_o[tt] = (part[0] + part[1]) + (part[2] + part[3]);
        }
        // the 16 lanes of a column add their shares of all the tile's tokens at once (as in the scan above)
        int n = TT;
#pragma unroll
        for (int off = GLA_KS / 2; off >= 1; off >>= 1) {
            const bool upper = (ks & off) != 0;
            if (n > 1) {
                const int half = n / 2;
#pragma unroll
                for (int i = 0; i < TT / 2; ++i)
                    if (i < half) {
                        const float mine = upper ? part_o[i + half] : part_o[i];
                        const float theirs = upper ? part_o[i] : part_o[i + half];
                        part_o[i] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
                    }
                n = half;
            } else {
                part_o[0] += __shfl_xor_sync(0xffffffffu, part_o[0], off);
            }
        }
        if (is_n && ks % SHARE == 0) nq_s[par][my_tt] = part_o[0];
        held = part_o[0];
    }
    __syncthreads();
    write_out((n_tok - 1) / TT * TT, par ^ 1);
    if (st != nullptr) {
#pragma unroll
        for (int ii = 0; ii < DPT; ++ii) {
            const int i = ks * DPT + ii;
            if (i < d) st[i] = S[ii];
        }
    }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :]); a warp per (token, head).  The weight is
// one vector of dv for all heads, or (w_per_head) one of H dv with a run per head; the gate is silu or (gate_sigmoid) the
// logistic function alone.
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ rows, int row_elems, int g_off,
                      const float* __restrict__ w, float eps, T* __restrict__ out, int n_tok, int H, int dv,
                      int w_per_head, int gate_sigmoid) {
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_dependents_launch();
    grid_dependency_wait();
    if (unit >= n_tok * H) return;
    const int t = unit / H, h = unit % H;
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const T* gate = rows != nullptr ? rows + (size_t)t * row_elems + g_off + h * dv : nullptr;
    T* dst = out + ((size_t)t * H + h) * dv;
    const float* wh = w_per_head ? w + (size_t)h * dv : w;
    for (int c = lane; c < dv; c += 32) {
        float y = src[c] * inv * wh[c];
        if (gate != nullptr) {
            const float gv = to_float(gate[c]);
            y *= (gate_sigmoid ? 1.0f : gv) / (1.0f + expf(-gv));
        }
        dst[c] = from_float<T>(y);
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT void janis_mixers_set_overlap(int on) { overlap_launches() = on ? 1 : 0; }

JANIS_EXPORT const char* janis_last_error() { return error_buffer(); }

template <typename T>
static int gla_scan_launch(const void* rows, const GlaRows& g, const float* decay, const int* seq_slot,
                           const int* seq_first_row, const int* seq_start, const int* seq_end, float* state, float* o_out,
                           int n_seq, cudaStream_t stream) {
    const dim3 grid(n_seq, g.H, (g.dv + GLA_COLS - 1) / GLA_COLS), block(GLA_COLS * GLA_KS);
#define JANIS_GLA_CASE(DPT)                                                                                            \
    if (g.d <= GLA_KS * DPT)                                                                                           \
        return launch_kernel("gla_scan", gla_scan_kernel<T, DPT>, grid, block, 0, stream, 1, (const T*)rows, g,        \
                             decay, seq_slot, seq_first_row, seq_start, seq_end, state, o_out);
    JANIS_GLA_CASE(4)
    JANIS_GLA_CASE(8)
    JANIS_GLA_CASE(16)
#undef JANIS_GLA_CASE
    return fail("gla_scan: key size %d is above %d", g.d, GLA_KS * 16);
}

JANIS_EXPORT int janis_gla_scan(const void* rows, int dtype, int row_elems, int q_off, int k_off, int v_off,
                                const void* z_rows, const void* z_bias, float* decay, int n_tok, const int* seq_slot,
                                const int* seq_first_row, const int* seq_start, const int* seq_end, float* state,
                                float* o_out, int n_seq, int H, int d, int dv, float q_scale, float tau, cudaStream_t stream) {
    if (n_seq <= 0 || n_tok <= 0) return 0;
    if (H <= 0 || d <= 0 || dv <= 0) return fail("gla_scan: sizes %d heads, %d x %d", H, d, dv);
    if (!(tau > 0.f)) return fail("gla_scan: tau must be positive");
    if (H > 65535) return fail("gla_scan: too many heads (%d)", H);
    GlaRows g;
    g.row_elems = row_elems; g.q_off = q_off; g.k_off = k_off; g.v_off = v_off;
    g.H = H; g.d = d; g.dv = dv; g.q_scale = q_scale; g.inv_tau = 1.0f / tau;
    const size_t n = (size_t)n_tok * H * d, want = (n + 255) / 256;
    const dim3 dgrid((unsigned)(want < 148 * 16 ? want : 148 * 16)), dblock(256);
    if (dtype == JANIS_F32) {
        if (launch_kernel("gla_decay", gla_decay_kernel<float>, dgrid, dblock, 0, stream, 1, (const float*)z_rows,
                          (const float*)z_bias, decay, n, H * d, g.inv_tau))
            return 1;
        return gla_scan_launch<float>(rows, g, decay, seq_slot, seq_first_row, seq_start, seq_end, state, o_out, n_seq, stream);
    }
    if (dtype == JANIS_BF16) {
        if (launch_kernel("gla_decay", gla_decay_kernel<bf16>, dgrid, dblock, 0, stream, 1, (const bf16*)z_rows,
                          (const bf16*)z_bias, decay, n, H * d, g.inv_tau))
            return 1;
        return gla_scan_launch<bf16>(rows, g, decay, seq_slot, seq_first_row, seq_start, seq_end, state, o_out, n_seq, stream);
    }
    return fail("gla_scan: unknown dtype %d", dtype);
}

template <typename T>
static int mlstm_scan_launch(const void* rows, const GlaRows& g, const float* coef, const int* seq_slot,
                             const int* seq_first_row, const int* seq_start, const int* seq_end, float* state_c,
                             float* state_n, float* o_out, int n_seq, cudaStream_t stream) {
    const dim3 grid(n_seq, g.H, (g.dv + GLA_COLS - 1) / GLA_COLS), block(MLSTM_THREADS);
#define JANIS_MLSTM_CASE(DPT)                                                                                          \
    if (g.d <= GLA_KS * DPT)                                                                                           \
        return launch_kernel("mlstm_scan", mlstm_scan_kernel<T, DPT>, grid, block, 0, stream, 1, (const T*)rows, g,    \
                             coef, seq_slot, seq_first_row, seq_start, seq_end, state_c, state_n, o_out);
    JANIS_MLSTM_CASE(4)
    JANIS_MLSTM_CASE(8)
    JANIS_MLSTM_CASE(16)
#undef JANIS_MLSTM_CASE
    return fail("mlstm_scan: key size %d is above %d", g.d, GLA_KS * 16);
}

// rows: the projected step (q [H, d], k [H, d], v [H, dv] at their offsets); z: float [n_tok, 2 H], the input gates'
// logits then the forget gates'; bias: float [2 H]; coef: float scratch [n_tok, H, 3]; the cache parts state_c
// [slots, H, dv, d], state_n [slots, H, ceil(dv / 8), d] and state_m [slots, H]; o_out float [n_tok, H dv].
JANIS_EXPORT int janis_mlstm_scan(const void* rows, int dtype, int row_elems, int q_off, int k_off, int v_off,
                                  const float* z, const float* bias, float cap, float* coef, int n_tok,
                                  const int* seq_slot, const int* seq_first_row, const int* seq_start, const int* seq_end,
                                  float* state_c, float* state_n, float* state_m, float* o_out, int n_seq, int H, int d,
                                  int dv, float q_scale, cudaStream_t stream) {
    if (n_seq <= 0 || n_tok <= 0) return 0;
    if (H <= 0 || d <= 0 || dv <= 0) return fail("mlstm_scan: sizes %d heads, %d x %d", H, d, dv);
    if (!(cap > 0.f)) return fail("mlstm_scan: the gates' cap must be positive");
    if (H > 65535) return fail("mlstm_scan: too many heads (%d)", H);
    if (launch_kernel("mlstm_gates", mlstm_gates_kernel<0>, dim3(n_seq, H), dim3(32), 0, stream, 1, z, bias, cap, H, seq_slot,
                      seq_first_row, seq_start, seq_end, state_m, coef))
        return 1;
    GlaRows g;
    g.row_elems = row_elems; g.q_off = q_off; g.k_off = k_off; g.v_off = v_off;
    g.H = H; g.d = d; g.dv = dv; g.q_scale = q_scale; g.inv_tau = 1.0f;
    if (dtype == JANIS_F32)
        return mlstm_scan_launch<float>(rows, g, coef, seq_slot, seq_first_row, seq_start, seq_end, state_c, state_n, o_out, n_seq, stream);
    if (dtype == JANIS_BF16)
        return mlstm_scan_launch<bf16>(rows, g, coef, seq_slot, seq_first_row, seq_start, seq_end, state_c, state_n, o_out, n_seq, stream);
    return fail("mlstm_scan: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_head_norm_gate(const float* o, const void* rows, int dtype, int row_elems, int g_off, const float* w,
                                      float eps, void* out, int T, int H, int dv, int w_per_head, int gate_sigmoid,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long units = (long long)T * H;
    const dim3 grid((unsigned)((units + 7) / 8)), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("head_norm_gate", head_norm_gate_kernel<float>, grid, block, 0, stream, 1, o, (const float*)rows,
                             row_elems, g_off, w, eps, (float*)out, T, H, dv, w_per_head, gate_sigmoid);
    if (dtype == JANIS_BF16)
        return launch_kernel("head_norm_gate", head_norm_gate_kernel<bf16>, grid, block, 0, stream, 1, o, (const bf16*)rows,
                             row_elems, g_off, w, eps, (bf16*)out, T, H, dv, w_per_head, gate_sigmoid);
    return fail("gla_scan: unknown dtype %d", dtype);
}
