// State-space mixers: a causal convolution per channel with silu, the selective scan, and the gated norm that
// follows the scan of the state-space-duality form.
//
//   conv:  x'[t, c] = silu(b[c] + sum_j w[c, K-1-j] x[t-j, c])      inputs before the sequence's start are zero;
//          the last K-1 inputs of a sequence are kept per slot, so that a later step goes on from them
//   scan:  S[c, n] <- exp(delta A) S[c, n] + delta u[c] B[n];   o[c] = sum_n S[c, n] C[n] + D u[c]
//          delta = softplus(dt + dt_bias); dt, A's row and D are indexed by c / ch_per_head, B and C by the group
//          c / ch_per_group.  With a state per (channel, n) in A and ch_per_head = 1 this is the selective scan of
//          Mamba; with one number per head in A it is the recurrence of its state-space-duality form.
//   norm:  y = rms_parts(o * silu(z)) * w over equal parts of a row
//
// delta, the decays, the state and o are float whatever the projections are stored in.  The state lives in the
// cache, [slots, C, N] floats per line: a step loads it, runs its tokens in order and writes it back; sequences
// without a slot (padding) start from zero and store nothing.
#include "common.cuh"

namespace janis {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// A state that remembers hundreds of tokens is multiplied by decays just below 1, where a float holds exp(x) to
// 6e-8 only and an error of one sign in every step adds up over the steps.  So the decay is kept as exp(x) - 1, which
// expm1f gives to its own last bit however small it is, and the step is S + (S (exp(x) - 1) + input): the bracket is
// small against S and its rounding does not count; what remains is the one rounding of the sum.
__device__ __forceinline__ float decay_minus_one(float x) { return expm1f(x); }
__device__ __forceinline__ float decayed(float S, float grow, float input) { return S + fmaf(S, grow, input); }

// ---------------------------------------------------------------------------
// convolution: a thread per channel and token (a CTA takes 256 channels of one token, or of 8 tokens in turn when
// the step has a thousand: launching a CTA costs more than a token's work); the taps that reach back before the step
// come from the slot's state.
// A sequence that brings one token (a decode step) has its kept inputs shifted by that token's threads; the second
// kernel serves the sequences that bring more, and is not launched when the caller says that none does.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const T* __restrict__ rows, int row_elems, int col_off, int C, int K,
                        const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ state,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_end, T* __restrict__ out, int n_tok, int tokens_per_cta, int act) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wk[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) wk[j] = j < K ? w[(size_t)c * K + K - 1 - j] : 0.f;      // wk[j]: the tap j tokens back
    const float b = bias != nullptr ? bias[c] : 0.f;
    const int t_end = min(n_tok, ((int)blockIdx.x + 1) * tokens_per_cta);
    for (int t = blockIdx.x * tokens_per_cta; t < t_end; ++t) {
        const int s = tok_seq[t], slot = seq_slot[s], i = t - seq_first_row[s];
        const bool alone = seq_end[s] - seq_start[s] == 1;   // the sequence's only token of the step: it shifts the kept inputs itself
        float* st = slot >= 0 ? state + (size_t)slot * max(K - 1, 1) * C : nullptr;
        float acc = b;
        float xs[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j >= K) break;
            const int idx = i - j;
            float x = 0.f;
            if (idx >= 0) x = to_float(rows[(size_t)(t - j) * row_elems + col_off + c]);
            else if (st != nullptr) x = st[(size_t)(K - 1 + idx) * C + c];
            xs[j] = x;
            acc = fmaf(wk[j], x, acc);
        }
        out[(size_t)t * C + c] = from_float<T>(act ? silu_f(acc) : acc);
        if (alone && st != nullptr) {                        // (i == 0: xs[j] is the input j tokens back; this thread alone touches (slot, c))
#pragma unroll
            for (int j = 0; j < 15; ++j) {
                if (j >= K - 1) break;
                st[(size_t)(K - 2 - j) * C + c] = xs[j];
            }
        }
    }
}

// the K-1 inputs a sequence ends the step with: a thread per (sequence, channel) reads them all, then writes
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ rows, int row_elems, int col_off, int C, int K, float* __restrict__ state,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_end) {
    const int s = blockIdx.x;
    grid_dependents_launch();
    const int slot = seq_slot[s], row0 = seq_first_row[s], n = seq_end[s] - seq_start[s];
    grid_dependency_wait();
    if (slot < 0 || n <= 1 || K <= 1) return;                // (a sequence's only token has shifted them in the convolution's kernel)
    float* st = state + (size_t)slot * (K - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[15];
#pragma unroll
        for (int jj = 0; jj < 15; ++jj) {
            if (jj >= K - 1) break;
            const int idx = n - (K - 1) + jj;
            keep[jj] = idx >= 0 ? to_float(rows[(size_t)(row0 + idx) * row_elems + col_off + c]) : st[(size_t)(jj + n) * C + c];
        }
#pragma unroll
        for (int jj = 0; jj < 15; ++jj) {
            if (jj >= K - 1) break;
            st[(size_t)jj * C + c] = keep[jj];
        }
    }
}

// ---------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------
struct ScanShape {
    int u_stride, u_off;           // u[t, c] = u_rows[t * u_stride + u_off + c]
    int bc_stride, b_off, c_off;   // B[t, group * N + n], C[t, group * N + n]
    int z_stride, z_off;           // the gate (when one is given)
    int gated;
    int C, N, cph, cpg, heads;
    int ln;                        // lanes that share a channel (a power of two up to 32); lane l holds states l SPL .. l SPL + SPL - 1
};

constexpr int SCAN_THREADS = 128;

// Step sizes once per (token, head), as floats: delta = softplus(dt + bias) and, where a head has one decay,
// exp(delta A) - 1.  (Left to the scan, every lane of a channel and every channel of a head would form them again.)
template <typename T>
__global__ void __launch_bounds__(256)
scan_steps_kernel(const T* __restrict__ dt_rows, int dt_stride, int dt_off, const float* __restrict__ dt_bias,
                  const float* __restrict__ A_head, float* __restrict__ delta, float* __restrict__ grow, int heads, size_t n) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / heads;
        const int h = (int)(i % heads);
        const float d = softplus_f(to_float(dt_rows[t * dt_stride + dt_off + h]) + dt_bias[h]);
        delta[i] = d;
        if (A_head != nullptr) grow[i] = decay_minus_one(d * A_head[h]);
    }
}

// SPL consecutive values as floats; VEC: loads of min(16, SPL * sizeof(T)) bytes (the address is aligned to that)
template <typename T, int SPL, bool VEC>
__device__ __forceinline__ void load_run(const T* __restrict__ p, float (&out)[SPL]) {
    if constexpr (VEC && sizeof(T) == 2 && SPL == 2) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
        out[0] = __uint_as_float(v << 16); out[1] = __uint_as_float(v & 0xffff0000u);
    } else if constexpr (VEC && sizeof(T) == 2 && SPL == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
        out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
    } else if constexpr (VEC && sizeof(T) == 2 && SPL % 8 == 0) {
#pragma unroll
        for (int q = 0; q < SPL / 8; ++q) {
            const uint4 v = reinterpret_cast<const uint4*>(p)[q];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                out[8 * q + 2 * i] = __uint_as_float(w[i] << 16);
                out[8 * q + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    } else if constexpr (VEC && sizeof(T) == 4 && SPL == 2) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        out[0] = v.x; out[1] = v.y;
    } else if constexpr (VEC && sizeof(T) == 4 && SPL % 4 == 0) {
#pragma unroll
        for (int i = 0; i < SPL / 4; ++i) {
            const float4 v = reinterpret_cast<const float4*>(p)[i];
            out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < SPL; ++k) out[k] = to_float(p[k]);
    }
}

// A CTA per (sequence, 128 / LN channels).  The inputs of a tile of TT tokens are asked for together, and those of
// the next tile while this one is computed (two sets of registers that take turns).  What a token costs beside its
// states (its step size, input, gate, the lanes' butterfly, the store) is shared by the SPL states of a lane, so the
// launch takes as few lanes a channel as still give every SM a CTA.
template <typename T, int SPL, bool PER_STATE, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const T* __restrict__ u_rows, const T* __restrict__ bc_rows, const T* __restrict__ z_rows,
                      const float* __restrict__ delta, const float* __restrict__ grow, const float* __restrict__ A,
                      const float* __restrict__ D, ScanShape g, const int* __restrict__ seq_slot,
                      const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                      const int* __restrict__ seq_end, float* __restrict__ state, void* __restrict__ out_raw) {
    constexpr int TT = SPL <= 2 ? 8 : (SPL <= 4 ? 4 : 2);          // tokens whose inputs are asked for together (deeper tiles measured slower)
    const int LN = g.ln, N = g.N, C = g.C;
    const int seq = blockIdx.x, tid = threadIdx.x, l = tid & (LN - 1), n0 = l * SPL;
    const int c_raw = blockIdx.y * (SCAN_THREADS / LN) + tid / LN;
    const bool live = c_raw < C;
    const int c = live ? c_raw : C - 1;
    const int head = c / g.cph, group = c / g.cpg;
    const bool whole = n0 + SPL <= N;                      // the lane's run lies inside the states (VEC: it does or is empty)
    const bool gated = g.gated != 0;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    const float Dh = D[head];
    float Areg[SPL];
#pragma unroll
    for (int k = 0; k < SPL; ++k) Areg[k] = (PER_STATE && n0 + k < N) ? A[(size_t)head * N + n0 + k] : 0.f;
    grid_dependency_wait();
    float S[SPL];
    float* st = slot >= 0 ? state + ((size_t)slot * C + c) * N : nullptr;
#pragma unroll
    for (int k = 0; k < SPL; ++k) S[k] = (st != nullptr && n0 + k < N) ? st[n0 + k] : 0.f;
    // the thread's columns in the sequence's first row
    const T* pu = u_rows + (size_t)row0 * g.u_stride + g.u_off + c;
    const T* pz = gated ? z_rows + (size_t)row0 * g.z_stride + g.z_off + c : nullptr;
    const T* pb = bc_rows + (size_t)row0 * g.bc_stride + g.b_off + group * N + n0;
    const int c_from_b = g.c_off - g.b_off;
    const float* pd = delta + (size_t)row0 * g.heads + head;
    const float* pg = PER_STATE ? nullptr : grow + (size_t)row0 * g.heads + head;
    T* out_t = reinterpret_cast<T*>(out_raw) + (size_t)row0 * C + c;
    float* out_f = reinterpret_cast<float*>(out_raw) + (size_t)row0 * C + c;
    struct Tile {
        float d[TT], gr[TT], u[TT], z[TT], B[TT][SPL], Cc[TT][SPL];
    };
    auto fetch = [&](int t0, Tile& x) {
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            const unsigned r = (unsigned)min(t0 + tt, n_tok - 1);
            x.d[tt] = pd[(size_t)r * g.heads];
            x.gr[tt] = PER_STATE ? 0.f : pg[(size_t)r * g.heads];
            x.u[tt] = to_float(pu[(size_t)r * g.u_stride]);
            x.z[tt] = gated ? to_float(pz[(size_t)r * g.z_stride]) : 0.f;
            const T* b = pb + (size_t)r * g.bc_stride;
            if (VEC) {
                if (whole) {
                    load_run<T, SPL, VEC>(b, x.B[tt]);
                    load_run<T, SPL, VEC>(b + c_from_b, x.Cc[tt]);
                } else {
#pragma unroll
                    for (int k = 0; k < SPL; ++k) x.B[tt][k] = x.Cc[tt][k] = 0.f;
                }
            } else {
#pragma unroll
                for (int k = 0; k < SPL; ++k) {
                    const bool in = n0 + k < N;
                    x.B[tt][k] = in ? to_float(b[k]) : 0.f;
                    x.Cc[tt][k] = in ? to_float(b[c_from_b + k]) : 0.f;
                }
            }
        }
    };
    auto run = [&](int t0, const Tile& x) {
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            const float dl = x.d[tt], du = dl * x.u[tt];
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int k = 0; k < SPL; ++k) {
                const float gr = PER_STATE ? decay_minus_one(dl * Areg[k]) : x.gr[tt];
                const float s_new = decayed(S[k], gr, du * x.B[tt][k]);
                S[k] = t0 + tt < n_tok ? s_new : S[k];         // (tokens beyond the sequence's end change nothing)
                if (k & 1) acc1 = fmaf(s_new, x.Cc[tt][k], acc1);
                else acc0 = fmaf(s_new, x.Cc[tt][k], acc0);
            }
            float acc = acc0 + acc1;
            for (int off = LN >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (l == 0 && live && t0 + tt < n_tok) {
                const float y = fmaf(Dh, x.u[tt], acc);
                const size_t at = (size_t)(unsigned)(t0 + tt) * C;
                if (gated) out_t[at] = from_float<T>(y * silu_f(x.z[tt]));
                else out_f[at] = y;
            }
        }
    };
    Tile ta, tb;
    fetch(0, ta);
    for (int t0 = 0; t0 < n_tok; t0 += 2 * TT) {
        if (t0 + TT < n_tok) fetch(t0 + TT, tb);
        run(t0, ta);
        if (t0 + TT >= n_tok) break;
        if (t0 + 2 * TT < n_tok) fetch(t0 + 2 * TT, ta);
        run(t0 + TT, tb);
    }
    if (st != nullptr && live) {
#pragma unroll
        for (int k = 0; k < SPL; ++k)
            if (n0 + k < N) st[n0 + k] = S[k];
    }
}

// The prompt form.  A token costs a channel's lanes little arithmetic, so the other form spends its time waiting
// for each token's inputs.  Here the B and C rows of a tile of 16 tokens, which every channel of the CTA reads, are
// copied into shared memory once (cp.async, 16 bytes a piece, the next tile's on their way while this one is
// computed: two buffers), and the tile's step sizes, inputs and gates, gathered per (token, channel), pass through
// registers a tile ahead and then through shared memory.  Conditions (the launcher checks them): the CTA's channels
// lie in one group of B and C, rows of B and C are whole 16-byte pieces at 16-byte offsets, no CTA is partly empty.
constexpr int SCAN_TS = 16;

__device__ __forceinline__ void scan_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

template <typename T, int SPL, bool PER_STATE, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_staged_kernel(const T* __restrict__ u_rows, const T* __restrict__ bc_rows, const T* __restrict__ z_rows,
                             const float* __restrict__ delta, const float* __restrict__ grow, const float* __restrict__ A,
                             const float* __restrict__ D, ScanShape g, const int* __restrict__ seq_slot,
                             const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                             const int* __restrict__ seq_end, float* __restrict__ state, void* __restrict__ out_raw) {
    extern __shared__ __align__(16) unsigned char scan_smem[];
    constexpr int TS = SCAN_TS, EPP = 16 / (int)sizeof(T);          // elements a 16-byte piece
    const int LN = g.ln, N = g.N, C = g.C, CPC = SCAN_THREADS / LN;
    T* bc_s = reinterpret_cast<T*>(scan_smem);                       // [2][TS][2][N]: a token's B, then its C
    float* sc_s = reinterpret_cast<float*>(scan_smem + (size_t)2 * TS * 2 * N * sizeof(T));      // [4][TS][CPC]: delta, grow, u, z
    const int seq = blockIdx.x, tid = threadIdx.x, l = tid & (LN - 1), n0 = l * SPL, j = tid / LN;
    const int c0 = blockIdx.y * CPC, c = c0 + j;
    const int head = c / g.cph, group = c0 / g.cpg;
    const bool whole = n0 + SPL <= N, gated = g.gated != 0;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    const float Dh = D[head];
    float Areg[SPL];
#pragma unroll
    for (int k = 0; k < SPL; ++k) Areg[k] = (PER_STATE && n0 + k < N) ? A[(size_t)head * N + n0 + k] : 0.f;
    grid_dependency_wait();
    float S[SPL];
    float* st = slot >= 0 ? state + ((size_t)slot * C + c) * N : nullptr;
#pragma unroll
    for (int k = 0; k < SPL; ++k) S[k] = (st != nullptr && n0 + k < N) ? st[n0 + k] : 0.f;
    const int pieces = N / EPP;                                      // 16-byte pieces of a row of B (and of C)
    const T* bsrc = bc_rows + (size_t)row0 * g.bc_stride + g.b_off + group * N;
    const int c_from_b = g.c_off - g.b_off;
    auto issue_bc = [&](int t0, int buf) {
        for (int p = tid; p < TS * 2 * pieces; p += SCAN_THREADS) {
            const int tt = p / (2 * pieces), q = p - tt * 2 * pieces, which = q >= pieces ? 1 : 0, i = q - which * pieces;
            const unsigned r = (unsigned)min(t0 + tt, n_tok - 1);
            scan_cp_async16(bc_s + ((size_t)(buf * TS + tt) * 2 + which) * N + i * EPP,
                            bsrc + (size_t)r * g.bc_stride + (which ? c_from_b : 0) + i * EPP);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    // the tile's scalars: element e = tid + i 128 is (token e / CPC, channel c0 + e % CPC)
    constexpr int SC = 4;                                            // TS CPC / 128 <= 4
    float sd[SC], sg[SC], su[SC], sz[SC];
    auto fetch_scalars = [&](int t0) {
#pragma unroll
        for (int i = 0; i < SC; ++i) {
            const int e = tid + i * SCAN_THREADS;
            sd[i] = sg[i] = su[i] = sz[i] = 0.f;
            if (e < TS * CPC) {
                const int tt = e / CPC, ch = c0 + e - tt * CPC;
                const size_t row = (size_t)(row0 + min(t0 + tt, n_tok - 1));
                const int h = ch / g.cph;
                sd[i] = delta[row * g.heads + h];
                if (!PER_STATE) sg[i] = grow[row * g.heads + h];
                su[i] = to_float(u_rows[row * g.u_stride + g.u_off + ch]);
                if (gated) sz[i] = to_float(z_rows[row * g.z_stride + g.z_off + ch]);
            }
        }
    };
    issue_bc(0, 0);
    fetch_scalars(0);
    T* out_t = reinterpret_cast<T*>(out_raw) + (size_t)row0 * C + c;
    float* out_f = reinterpret_cast<float*>(out_raw) + (size_t)row0 * C + c;
    int buf = 0;
    for (int t0 = 0; t0 < n_tok; t0 += TS, buf ^= 1) {
        __syncthreads();                                             // the tile before has been read
#pragma unroll
        for (int i = 0; i < SC; ++i) {
            const int e = tid + i * SCAN_THREADS;
            if (e < TS * CPC) {
                sc_s[e] = sd[i];
                sc_s[TS * CPC + e] = sg[i];
                sc_s[2 * TS * CPC + e] = su[i];
                sc_s[3 * TS * CPC + e] = sz[i];
            }
        }
        const bool more = t0 + TS < n_tok;
        if (more) {
            issue_bc(t0 + TS, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        if (more) fetch_scalars(t0 + TS);
        const int tt_n = min(TS, n_tok - t0);
        for (int tt = 0; tt < tt_n; ++tt) {
            const float dl = sc_s[tt * CPC + j], grh = sc_s[TS * CPC + tt * CPC + j], uu = sc_s[2 * TS * CPC + tt * CPC + j];
            const float du = dl * uu;
            float Bv[SPL], Cv[SPL];
            const T* brow = bc_s + ((size_t)(buf * TS + tt) * 2) * N + n0;
            if (VEC) {
                if (whole) {
                    load_run<T, SPL, VEC>(brow, Bv);
                    load_run<T, SPL, VEC>(brow + N, Cv);
                } else {
#pragma unroll
                    for (int k = 0; k < SPL; ++k) Bv[k] = Cv[k] = 0.f;
                }
            } else {
#pragma unroll
                for (int k = 0; k < SPL; ++k) {
                    const bool in = n0 + k < N;
                    Bv[k] = in ? to_float(brow[k]) : 0.f;
                    Cv[k] = in ? to_float(brow[N + k]) : 0.f;
                }
            }
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int k = 0; k < SPL; ++k) {
                const float gr = PER_STATE ? decay_minus_one(dl * Areg[k]) : grh;
                S[k] = decayed(S[k], gr, du * Bv[k]);
                if (k & 1) acc1 = fmaf(S[k], Cv[k], acc1);
                else acc0 = fmaf(S[k], Cv[k], acc0);
            }
            float acc = acc0 + acc1;
            for (int off = LN >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (l == 0) {
                const float y = fmaf(Dh, uu, acc);
                const size_t at = (size_t)(unsigned)(t0 + tt) * C;
                if (gated) out_t[at] = from_float<T>(y * silu_f(sc_s[3 * TS * CPC + tt * CPC + j]));
                else out_f[at] = y;
            }
        }
    }
    if (st != nullptr) {
#pragma unroll
        for (int k = 0; k < SPL; ++k)
            if (n0 + k < N) st[n0 + k] = S[k];
    }
}

// y[t, part] = x / sqrt(mean(x^2) + eps) * w with x = o * silu(z): a CTA per (token, part)
template <typename T>
__global__ void __launch_bounds__(256)
gate_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ rows, int row_elems, int z_off,
                       const float* __restrict__ w, float eps, T* __restrict__ out, int C, int per) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, c0 = blockIdx.y * per;
    grid_dependents_launch();
    grid_dependency_wait();
    const float* src = o + (size_t)t * C + c0;
    const T* z = rows + (size_t)t * row_elems + z_off + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float v = src[i] * silu_f(to_float(z[i]));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)per + eps);
    T* dst = out + (size_t)t * C + c0;
    for (int i = threadIdx.x; i < per; i += blockDim.x)
        dst[i] = from_float<T>(src[i] * silu_f(to_float(z[i])) * inv * w[c0 + i]);
}

}  // namespace janis

using namespace janis;

template <typename T>
static int conv_launch(const void* rows, int row_elems, int col_off, int C, int K, const float* w, const float* bias,
                       float* state, const int* tok_seq, const int* seq_slot, const int* seq_first_row,
                       const int* seq_start, const int* seq_end, int n_tok, int n_seq, int one_token, void* out,
                       int act, cudaStream_t stream) {
    const int by = (C + 255) / 256, tpc = n_tok >= 1024 ? 8 : 1;
    if (by > 65535) return fail("causal_conv_silu: too many channels (%d)", C);
    if (launch_kernel("causal_conv_silu", causal_conv_silu_kernel<T>, dim3((n_tok + tpc - 1) / tpc, by), dim3(256), 0, stream, 1,
                      (const T*)rows, row_elems, col_off, C, K, w, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                      seq_end, (T*)out, n_tok, tpc, act))
        return 1;
    if (K <= 1 || one_token) return 0;
    return launch_kernel("conv_state_update", conv_state_update_kernel<T>, dim3(n_seq, by < 64 ? by : 64), dim3(256), 0, stream, 1,
                         (const T*)rows, row_elems, col_off, C, K, state, seq_slot, seq_first_row, seq_start, seq_end);
}

JANIS_EXPORT int janis_causal_conv_silu(const void* rows, int dtype, int row_elems, int col_off, int C, int K,
                                        const float* w, const float* bias, float* state, const int* tok_seq,
                                        const int* seq_slot, const int* seq_first_row, const int* seq_start,
                                        const int* seq_end, int n_tok, int n_seq, int one_token, void* out,
                                        int act, cudaStream_t stream) {
    if (n_tok <= 0 || n_seq <= 0) return 0;
    if (K < 1 || K > 16) return fail("causal_conv_silu: %d taps (1 to 16 are taken)", K);
    if (C <= 0 || col_off < 0 || col_off + C > row_elems) return fail("causal_conv_silu: channels %d at %d do not fit rows of %d", C, col_off, row_elems);
    if (dtype == JANIS_F32)
        return conv_launch<float>(rows, row_elems, col_off, C, K, w, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                                  seq_end, n_tok, n_seq, one_token, out, act, stream);
    if (dtype == JANIS_BF16)
        return conv_launch<bf16>(rows, row_elems, col_off, C, K, w, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                                 seq_end, n_tok, n_seq, one_token, out, act, stream);
    return fail("causal_conv_silu: unknown dtype %d", dtype);
}

// The kept inputs of a filter brought up to date from rows that another kernel filtered (one that shifts them itself for
// sequences that bring a single token).
JANIS_EXPORT int janis_conv_state_update(const void* rows, int dtype, int row_elems, int col_off, int C, int K, float* state,
                                         const int* seq_slot, const int* seq_first_row, const int* seq_start,
                                         const int* seq_end, int n_seq, cudaStream_t stream) {
    if (n_seq <= 0 || K <= 1) return 0;
    if (K > 16) return fail("conv_state_update: %d taps (1 to 16 are taken)", K);
    if (C <= 0 || col_off < 0 || col_off + C > row_elems) return fail("conv_state_update: channels %d at %d do not fit rows of %d", C, col_off, row_elems);
    const int by = (C + 255) / 256;
    const dim3 grid(n_seq, by < 64 ? by : 64), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("conv_state_update", conv_state_update_kernel<float>, grid, block, 0, stream, 1, (const float*)rows,
                             row_elems, col_off, C, K, state, seq_slot, seq_first_row, seq_start, seq_end);
    if (dtype == JANIS_BF16)
        return launch_kernel("conv_state_update", conv_state_update_kernel<bf16>, grid, block, 0, stream, 1, (const bf16*)rows,
                             row_elems, col_off, C, K, state, seq_slot, seq_first_row, seq_start, seq_end);
    return fail("conv_state_update: unknown dtype %d", dtype);
}

template <typename T, bool PER_STATE>
static int scan_launch(const void* u, const void* bc, const void* z, const float* delta, const float* grow, const float* A,
                       const float* D, ScanShape g, int spl, bool vec, size_t staged_bytes, const int* seq_slot,
                       const int* seq_first_row, const int* seq_start, const int* seq_end, int n_seq, float* state, void* out,
                       cudaStream_t stream) {
    const int per_cta = SCAN_THREADS / g.ln;
    const dim3 grid(n_seq, (g.C + per_cta - 1) / per_cta), block(SCAN_THREADS);
    if (staged_bytes > 0) {
#define JANIS_SCAN_STAGED(SPL, VEC)                                                                                    \
    {                                                                                                                  \
        static size_t most = 0;                                                                                        \
        if (staged_bytes > most) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(selective_scan_staged_kernel<T, SPL, PER_STATE, VEC>,                 \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged_bytes);      \
            if (e != cudaSuccess) return fail("selective_scan: shared memory of %zu bytes refused: %s", staged_bytes, cudaGetErrorString(e)); \
            most = staged_bytes;                                                                                       \
        }                                                                                                              \
        return launch_kernel("selective_scan", selective_scan_staged_kernel<T, SPL, PER_STATE, VEC>, grid, block,      \
                             staged_bytes, stream, 1, (const T*)u, (const T*)bc, (const T*)z, delta, grow, A, D, g,     \
                             seq_slot, seq_first_row, seq_start, seq_end, state, out);                                  \
    }
        if (vec) {
            if (spl == 2) JANIS_SCAN_STAGED(2, true)
            if (spl == 4) JANIS_SCAN_STAGED(4, true)
            if (spl == 8) JANIS_SCAN_STAGED(8, true)
            if (spl == 16) JANIS_SCAN_STAGED(16, true)
        }
        if (spl <= 1) JANIS_SCAN_STAGED(1, false)
        if (spl <= 2) JANIS_SCAN_STAGED(2, false)
        if (spl <= 3) JANIS_SCAN_STAGED(3, false)
        if (spl <= 4) JANIS_SCAN_STAGED(4, false)
        if (spl <= 6) JANIS_SCAN_STAGED(6, false)
        if (spl <= 8) JANIS_SCAN_STAGED(8, false)
        if (spl <= 16) JANIS_SCAN_STAGED(16, false)
#undef JANIS_SCAN_STAGED
    }
#define JANIS_SCAN_LAUNCH(SPL, VEC)                                                                                    \
    return launch_kernel("selective_scan", selective_scan_kernel<T, SPL, PER_STATE, VEC>, grid, block, 0, stream, 1,    \
                         (const T*)u, (const T*)bc, (const T*)z, delta, grow, A, D, g, seq_slot, seq_first_row,          \
                         seq_start, seq_end, state, out);
    if (vec) {
        if (spl == 2) { JANIS_SCAN_LAUNCH(2, true) }
        if (spl == 4) { JANIS_SCAN_LAUNCH(4, true) }
        if (spl == 8) { JANIS_SCAN_LAUNCH(8, true) }
        if (spl == 16) { JANIS_SCAN_LAUNCH(16, true) }
    }
    if (spl <= 1) { JANIS_SCAN_LAUNCH(1, false) }
    if (spl <= 2) { JANIS_SCAN_LAUNCH(2, false) }
    if (spl <= 3) { JANIS_SCAN_LAUNCH(3, false) }
    if (spl <= 4) { JANIS_SCAN_LAUNCH(4, false) }
    if (spl <= 6) { JANIS_SCAN_LAUNCH(6, false) }
    if (spl <= 8) { JANIS_SCAN_LAUNCH(8, false) }
    if (spl <= 16) { JANIS_SCAN_LAUNCH(16, false) }
#undef JANIS_SCAN_LAUNCH
    return fail("selective_scan: %d states a channel are above %d", g.N, 32 * 16);
}

JANIS_EXPORT long long janis_selective_scan_scratch(int n_tok, int heads) { return 2LL * n_tok * heads; }

static int scan_lanes_forced = 0;      // lanes a channel fixed by a test or a tuning run (0: chosen per launch)

JANIS_EXPORT void janis_selective_scan_set_lanes(int lanes) { scan_lanes_forced = lanes; }

static int scan_form_forced = 0;       // 0: the prompt form with its tiles in shared memory where it fits and pays; 1: never; 2: wherever it fits (tests)

JANIS_EXPORT void janis_selective_scan_set_form(int form) { scan_form_forced = form; }

JANIS_EXPORT int janis_selective_scan(const void* u, int dtype, int u_stride, int u_off, const void* dt, int dt_stride,
                                      int dt_off, const float* dt_bias, const float* A, int a_per_state, const void* bc,
                                      int bc_stride, int b_off, int c_off, const float* D, const void* z, int z_stride,
                                      int z_off, const int* seq_slot, const int* seq_first_row, const int* seq_start,
                                      const int* seq_end, int n_seq, float* state, void* out, int C, int N, int cph,
                                      int cpg, int n_tok, float* scratch, cudaStream_t stream) {
    if (n_seq <= 0 || n_tok <= 0) return 0;
    if (C <= 0 || N <= 0 || cph <= 0 || cpg <= 0 || C % cph || C % cpg)
        return fail("selective_scan: %d channels, %d states, %d a head, %d a group", C, N, cph, cpg);
    if (scratch == nullptr) return fail("selective_scan: no scratch for the step sizes");
    ScanShape g;
    g.u_stride = u_stride; g.u_off = u_off; g.bc_stride = bc_stride; g.b_off = b_off; g.c_off = c_off;
    g.z_stride = z_stride; g.z_off = z_off; g.gated = z != nullptr ? 1 : 0;
    g.C = C; g.N = N; g.cph = cph; g.cpg = cpg; g.heads = C / cph;
    // Lanes a channel and states a lane.  What a token costs beside its states is shared by the states of a lane, so a
    // prompt takes the fewest lanes that still give the launch some 256 CTAs, among the pairs that waste the fewest
    // places (else the most lanes among them).  A step of one token a sequence only loads and stores the state: it
    // takes about N / 2 lanes, up to 16.  (B200, 4,608 channels, one sequence of 2,048 tokens: 128 states 1.28 ms
    // with 8 lanes, 2.16 with 16, 3.04 with 32; 16 states 1.35 ms with 4 lanes, 1.00 with 8, 1.71 with 16.  Eight
    // sequences of one token: 128 states 40 us with 8 lanes, 30 with 16, 51 with 32; 16 states 35, 33, 42 us.)
    static const int spls[7] = {1, 2, 3, 4, 6, 8, 16};
    auto spl_for = [&](int ln) {
        for (int i = 0; i < 7; ++i)
            if (ln * spls[i] >= N) return spls[i];
        return 0;
    };
    int best = 1 << 30;
    for (int ln = 4; ln <= 32; ln <<= 1)
        if (spl_for(ln) && ln * spl_for(ln) < best) best = ln * spl_for(ln);
    if (best == 1 << 30) return fail("selective_scan: %d states a channel are above %d", N, 32 * 16);
    int best_ln = 0, best_spl = 0;
    if (n_tok == n_seq) {
        int ln = 4;
        while (ln * 2 <= 16 && ln * 2 <= N / 2) ln *= 2;
        while (!spl_for(ln)) ln *= 2;
        best_ln = ln;
    } else {
        for (int ln = 4; ln <= 32; ln <<= 1)
            if (spl_for(ln) && ln * spl_for(ln) == best) {
                best_ln = ln;
                if ((long long)n_seq * ((C * ln + SCAN_THREADS - 1) / SCAN_THREADS) >= 256) break;
            }
    }
    best_spl = spl_for(best_ln);
    if (scan_lanes_forced && spl_for(scan_lanes_forced)) {
        best_ln = scan_lanes_forced;
        best_spl = spl_for(best_ln);
    }
    g.ln = best_ln;
    const size_t esz = dtype == JANIS_F32 ? 4 : 2, run = (size_t)best_spl * esz < 16 ? (size_t)best_spl * esz : 16;
    const bool vec = (best_spl == 2 || best_spl == 4 || best_spl == 8 || best_spl == 16) && N % best_spl == 0 && b_off % best_spl == 0 &&
                     c_off % best_spl == 0 && bc_stride % best_spl == 0 && ((uintptr_t)bc % run) == 0 &&
                     ((size_t)bc_stride * esz) % run == 0 && ((size_t)b_off * esz) % run == 0 && ((size_t)c_off * esz) % run == 0;
    // the prompt form where its conditions hold (see the kernel): 0 bytes means the other form
    size_t staged_bytes = 0;
    {
        const int cpc = SCAN_THREADS / best_ln;
        const size_t row_bytes = (size_t)N * esz;
        // (with few states a token's rows are small and the tile's two barriers cost more than the copies save: 4,608
        // channels, 2,048 tokens, 16 states 1.6 ms against 1.0 in the other form; 128 states 0.96 against 1.28)
        const bool fits = n_tok > n_seq && scan_form_forced != 1 && (N >= 64 || scan_form_forced == 2) && C % cpc == 0 && cpg % cpc == 0 && row_bytes % 16 == 0 &&
                          ((size_t)bc_stride * esz) % 16 == 0 && ((size_t)b_off * esz) % 16 == 0 && ((size_t)c_off * esz) % 16 == 0 &&
                          ((uintptr_t)bc & 15) == 0 && SCAN_TS * cpc <= 4 * SCAN_THREADS;
        const size_t bytes = (size_t)2 * SCAN_TS * 2 * row_bytes + (size_t)4 * SCAN_TS * cpc * sizeof(float);
        if (fits && bytes <= 96 * 1024) staged_bytes = bytes;
    }
    float* delta = scratch;
    float* grow = scratch + (size_t)n_tok * g.heads;
    const size_t n = (size_t)n_tok * g.heads, want = (n + 255) / 256;
    const dim3 sgrid((unsigned)(want < 148 * 8 ? want : 148 * 8)), sblock(256);
    const float* A_head = a_per_state ? nullptr : A;
    if (dtype == JANIS_F32) {
        if (launch_kernel("scan_steps", scan_steps_kernel<float>, sgrid, sblock, 0, stream, 1, (const float*)dt, dt_stride, dt_off,
                          dt_bias, A_head, delta, grow, g.heads, n))
            return 1;
        return a_per_state ? scan_launch<float, true>(u, bc, z, delta, grow, A, D, g, best_spl, vec, staged_bytes, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream)
                           : scan_launch<float, false>(u, bc, z, delta, grow, A, D, g, best_spl, vec, staged_bytes, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream);
    }
    if (dtype == JANIS_BF16) {
        if (launch_kernel("scan_steps", scan_steps_kernel<bf16>, sgrid, sblock, 0, stream, 1, (const bf16*)dt, dt_stride, dt_off,
                          dt_bias, A_head, delta, grow, g.heads, n))
            return 1;
        return a_per_state ? scan_launch<bf16, true>(u, bc, z, delta, grow, A, D, g, best_spl, vec, staged_bytes, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream)
                           : scan_launch<bf16, false>(u, bc, z, delta, grow, A, D, g, best_spl, vec, staged_bytes, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream);
    }
    return fail("selective_scan: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_gate_group_norm(const float* o, const void* rows, int dtype, int row_elems, int z_off, const float* w,
                                       float eps, int n_groups, void* out, int T, int C, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_groups <= 0 || C % n_groups || n_groups > 65535) return fail("gate_group_norm: %d channels in %d parts", C, n_groups);
    const dim3 grid(T, n_groups), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("gate_group_norm", gate_group_norm_kernel<float>, grid, block, 0, stream, 1, o, (const float*)rows,
                             row_elems, z_off, w, eps, (float*)out, C, C / n_groups);
    if (dtype == JANIS_BF16)
        return launch_kernel("gate_group_norm", gate_group_norm_kernel<bf16>, grid, block, 0, stream, 1, o, (const bf16*)rows,
                             row_elems, z_off, w, eps, (bf16*)out, C, C / n_groups);
    return fail("gate_group_norm: unknown dtype %d", dtype);
}
