// What stands between an attention's projections and its scores, for mixers that filter, norm or compress their
// queries, keys and values before they cache them, and small products that run head by head.
//
//   qkv_conv_norm_store   a short causal filter over time on every channel of q | k | v (taps that reach back before
//                         the step come from the slot's kept inputs), an RMS norm over the whole of q and over the
//                         whole of k (one mean over all heads, a weight vector each), every value head divided by its
//                         own root mean square, q written to rows of its own, k and v into the paged cache line.
//                         Each of the steps is optional.
//   latent_rotate_store   a compressed key/value row [c | r]: c RMS-normed with a weight, r turned by the token's
//                         position (neighbouring pairs 2i, 2i + 1 of its first `rot` features; sine and cosine times an amplitude), the two written
//                         side by side as the one "key" of a cache line with a single head; the turned part of every
//                         query head is turned the same way and written behind the place of its absorbed part.
//   head_linear           out[t, h, :] = W[h] x[t, h, :] for every head h: a product per head with its own matrix.
//
// All sums, roots and angles are float whatever is stored.  A sum's order depends on the sizes alone.
#include "common.cuh"

#include <math_constants.h>

namespace janis {

constexpr int PREP_THREADS = 256;
constexpr int PREP_MANY_ROWS = 1024;      // from here on a CTA of the wide kernel takes four rows, or two

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
qkv_conv_norm_store_kernel(const T* __restrict__ rows, int row_elems, int H, int G, int d, int dv, int K,
                           const float* __restrict__ conv_w, float* __restrict__ conv_state,
                           const float* __restrict__ wq, const float* __restrict__ wk, int v_unit, float eps,
                           const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                           const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                           const int* __restrict__ seq_start, const int* __restrict__ seq_end, T* __restrict__ q_out,
                           T* __restrict__ kpool, T* __restrict__ vpool, const int* __restrict__ page_table,
                           int table_stride) {
    extern __shared__ float prep_smem[];
    const int Cq = H * d, Ck = G * d, Cv = G * dv, C = Cq + Ck + Cv;
    float* x_s = prep_smem;                 // the token's filtered row
    float* inv_s = x_s + C;                 // 1 / rms of q, of k, of each value head
    float* scratch = inv_s + 2 + G;         // 32 floats for block sums
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = PREP_THREADS >> 5;
    grid_dependents_launch();
    const int s = tok_seq[t], slot = seq_slot[s], pos = tok_pos[t], i = t - seq_first_row[s];
    const bool alone = seq_end[s] - seq_start[s] == 1;      // the sequence's only token of the step shifts the kept inputs itself
    grid_dependency_wait();
    const T* row = rows + (size_t)t * row_elems;
    if (conv_w != nullptr && K > 1) {
        float* st = slot >= 0 ? conv_state + (size_t)slot * (K - 1) * C : nullptr;
        for (int c = tid; c < C; c += PREP_THREADS) {
            float acc = 0.f, xs[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j >= K) break;
                const int idx = i - j;                      // the input j tokens back
                float x = 0.f;
                if (idx >= 0) x = to_float(rows[(size_t)(t - j) * row_elems + c]);
                else if (st != nullptr) x = st[(size_t)(K - 1 + idx) * C + c];
                xs[j] = x;
                acc = fmaf(conv_w[(size_t)c * K + K - 1 - j], x, acc);
            }
            x_s[c] = acc;
            if (alone && st != nullptr) {
#pragma unroll
                for (int j = 0; j < 15; ++j) {
                    if (j >= K - 1) break;
                    st[(size_t)(K - 2 - j) * C + c] = xs[j];
                }
            }
        }
    } else {
        const float w0 = conv_w != nullptr ? 1.f : 0.f;     // (a filter of one tap scales the channel)
        for (int c = tid; c < C; c += PREP_THREADS) {
            const float x = to_float(row[c]);
            x_s[c] = w0 != 0.f ? x * conv_w[c] : x;
        }
    }
    __syncthreads();
    {
        float sq = 0.f, sk = 0.f;
        if (wq != nullptr)
            for (int c = tid; c < Cq; c += PREP_THREADS) sq = fmaf(x_s[c], x_s[c], sq);
        if (wk != nullptr)
            for (int c = tid; c < Ck; c += PREP_THREADS) sk = fmaf(x_s[Cq + c], x_s[Cq + c], sk);
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        if (tid == 0) {
            inv_s[0] = wq != nullptr ? 1.f / sqrtf(sq / (float)Cq + eps) : 1.f;
            inv_s[1] = wk != nullptr ? 1.f / sqrtf(sk / (float)Ck + eps) : 1.f;
        }
        for (int g = warp; g < G; g += nwarp) {
            float sv = 0.f;
            if (v_unit)
                for (int c = lane; c < dv; c += 32) {
                    const float v = x_s[Cq + Ck + g * dv + c];
                    sv = fmaf(v, v, sv);
                }
            sv = warp_sum(sv);
            if (lane == 0) inv_s[2 + g] = v_unit ? 1.f / sqrtf(sv / (float)dv + eps) : 1.f;
        }
    }
    __syncthreads();
    T* q_row = q_out + (size_t)t * Cq;
    const float iq = inv_s[0], ik = inv_s[1];
    for (int c = tid; c < Cq; c += PREP_THREADS) q_row[c] = from_float<T>(wq != nullptr ? x_s[c] * iq * wq[c] : x_s[c]);
    if (slot < 0) return;                                   // a padding row: its keys and values are stored nowhere
    const int page = page_table[(size_t)slot * table_stride + pos / JANIS_PAGE];
    T* kdst = kpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * d;
    T* vdst = vpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * dv;
    for (int c = tid; c < Ck; c += PREP_THREADS) {
        const float v = wk != nullptr ? x_s[Cq + c] * ik * wk[c] : x_s[Cq + c];
        kdst[(size_t)(c / d) * JANIS_PAGE * d + c % d] = from_float<T>(v);
    }
    for (int c = tid; c < Cv; c += PREP_THREADS) {
        const int g = c / dv;
        vdst[(size_t)g * JANIS_PAGE * dv + c % dv] = from_float<T>(x_s[Cq + Ck + c] * inv_s[2 + g]);
    }
}

// The same with 16 bytes a load and a store, for sizes that allow it (heads that are multiples of 16 bytes, up to four
// taps known when the kernel is compiled).  A CTA takes TOK neighbouring rows of the step.  A thread keeps the filter of
// its 16 bytes of channels in registers for all of them, and the step's last KT - 1 rows too, so a row is read once (and
// KT - 1 rows before the CTA's first) and the filter once per CTA; where a tap reaches back before its sequence's part
// of the step it takes the slot's kept input (or zero) instead.  The filtered rows wait in shared memory for the sums of
// squares, which start in the filter's registers.  The sums' order depends on the sizes alone, not on TOK.
// KT: the taps (1: no filter, or one tap that scales the channel).
template <typename T, int KT, int TOK>
__global__ void __launch_bounds__(PREP_THREADS)
qkv_conv_norm_store_vec_kernel(const T* __restrict__ rows, int row_elems, int n_tok, int H, int G, int d, int dv,
                               const float* __restrict__ conv_w, float* __restrict__ conv_state,
                               const float* __restrict__ wq, const float* __restrict__ wk, int v_unit, float eps,
                               const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                               const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                               const int* __restrict__ seq_start, const int* __restrict__ seq_end, T* __restrict__ q_out,
                               T* __restrict__ kpool, T* __restrict__ vpool, const int* __restrict__ page_table,
                               int table_stride) {
    constexpr int V = Vec16<T>::N, NW = PREP_THREADS / 32, KB = KT > 1 ? KT - 1 : 1;
    extern __shared__ float prep_smem[];
    const int Cq = H * d, Ck = G * d, Cv = G * dv, C = Cq + Ck + Cv;
    float* x_s = prep_smem;                         // TOK filtered rows
    float* inv_s = x_s + (size_t)TOK * C;           // per row: 1 / rms of q, of k, of each value head
    float* scratch = inv_s + TOK * (2 + G);         // per warp and row: the partial sums of q and of k
    const int t0 = blockIdx.x * TOK, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_here = min(TOK, n_tok - t0);
    grid_dependents_launch();
    int in_seq[TOK], slot[TOK];
    bool alone[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        in_seq[k] = 0, slot[k] = -1, alone[k] = false;
        if (k < n_here) {
            const int s = tok_seq[t0 + k];
            slot[k] = seq_slot[s];
            in_seq[k] = t0 + k - seq_first_row[s];
            alone[k] = seq_end[s] - seq_start[s] == 1;      // the sequence's only token of the step shifts the kept inputs itself
        }
    }
    grid_dependency_wait();
    float sq[TOK], sk[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) sq[k] = sk[k] = 0.f;
    for (int c0 = tid * V; c0 < C; c0 += PREP_THREADS * V) {
        float w[V * KT], back[KB][V];                       // back[j - 1]: the step's row j before the one at hand
        if (conv_w != nullptr) {
#pragma unroll
            for (int e = 0; e < V * KT; e += 4) Vec16<float>::load(conv_w + (size_t)c0 * KT + e, w + e);
        }
#pragma unroll
        for (int j = 1; j < KT; ++j) {
            if (t0 - j >= 0) {
                Vec16<T>::load(rows + (size_t)(t0 - j) * row_elems + c0, back[j - 1]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) back[j - 1][e] = 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            if (k >= n_here) break;
            float xs[KT][V], acc[V];
            float* st = (KT > 1 && slot[k] >= 0) ? conv_state + (size_t)slot[k] * (KT - 1) * C : nullptr;
            Vec16<T>::load(rows + (size_t)(t0 + k) * row_elems + c0, xs[0]);
#pragma unroll
            for (int j = 1; j < KT; ++j) {
                const int idx = in_seq[k] - j;              // the input j tokens back
                if (idx >= 0) {
#pragma unroll
                    for (int e = 0; e < V; ++e) xs[j][e] = back[j - 1][e];
                } else if (st != nullptr) {
#pragma unroll
                    for (int e = 0; e < V; e += 4) Vec16<float>::load(st + (size_t)(KT - 1 + idx) * C + c0 + e, xs[j] + e);
                } else {
#pragma unroll
                    for (int e = 0; e < V; ++e) xs[j][e] = 0.f;
                }
            }
            if (conv_w != nullptr) {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < KT; ++j) a = fmaf(w[e * KT + KT - 1 - j], xs[j][e], a);
                    acc[e] = KT > 1 ? a : xs[0][e] * w[e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = xs[0][e];
            }
            if (KT > 1 && alone[k] && st != nullptr) {
#pragma unroll
                for (int j = 0; j < KT - 1; ++j)
#pragma unroll
                    for (int e = 0; e < V; e += 4) Vec16<float>::store(st + (size_t)(KT - 2 - j) * C + c0 + e, xs[j] + e);
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < V; ++e) ss = fmaf(acc[e], acc[e], ss);
#pragma unroll
            for (int e = 0; e < V; e += 4) Vec16<float>::store(x_s + (size_t)k * C + c0 + e, acc + e);
            if (c0 < Cq) sq[k] += ss;
            else if (c0 < Cq + Ck) sk[k] += ss;
#pragma unroll
            for (int j = KT - 2; j >= 1; --j)
#pragma unroll
                for (int e = 0; e < V; ++e) back[j][e] = back[j - 1][e];
            if (KT > 1) {
#pragma unroll
                for (int e = 0; e < V; ++e) back[0][e] = xs[0][e];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        const float a = warp_sum(sq[k]), b = warp_sum(sk[k]);
        if (lane == 0) scratch[(warp * TOK + k) * 2] = a, scratch[(warp * TOK + k) * 2 + 1] = b;
    }
    __syncthreads();                                        // (the filtered rows are whole now, too)
    if (tid < 2 * TOK) {
        const int k = tid >> 1, which = tid & 1;
        float tot = 0.f;
        for (int wp = 0; wp < NW; ++wp) tot += scratch[(wp * TOK + k) * 2 + which];
        const float* wt = which ? wk : wq;
        inv_s[k * (2 + G) + which] = wt != nullptr ? 1.f / sqrtf(tot / (float)(which ? Ck : Cq) + eps) : 1.f;
    }
    for (int p = warp; p < n_here * G; p += NW) {
        const int k = p / G, g = p % G;
        float sv = 0.f;
        if (v_unit)
            for (int c = lane; c < dv; c += 32) {
                const float v = x_s[(size_t)k * C + Cq + Ck + g * dv + c];
                sv = fmaf(v, v, sv);
            }
        sv = warp_sum(sv);
        if (lane == 0) inv_s[k * (2 + G) + 2 + g] = v_unit ? 1.f / sqrtf(sv / (float)dv + eps) : 1.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        if (k >= n_here) break;
        const float* xr = x_s + (size_t)k * C;
        const float iq = inv_s[k * (2 + G)], ik = inv_s[k * (2 + G) + 1];
        T* q_row = q_out + (size_t)(t0 + k) * Cq;
        int page = 0;
        const int pos = tok_pos[t0 + k];
        if (slot[k] >= 0) page = page_table[(size_t)slot[k] * table_stride + pos / JANIS_PAGE];
        T* kdst = kpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * d;
        T* vdst = vpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * dv;
        for (int c0 = tid * V; c0 < C; c0 += PREP_THREADS * V) {
            float y[V], w[V];
            T* dst;
#pragma unroll
            for (int e = 0; e < V; e += 4) Vec16<float>::load(xr + c0 + e, y + e);
            if (c0 < Cq) {
                dst = q_row + c0;
                if (wq != nullptr) {
#pragma unroll
                    for (int e = 0; e < V; e += 4) Vec16<float>::load(wq + c0 + e, w + e);
#pragma unroll
                    for (int e = 0; e < V; ++e) y[e] = y[e] * iq * w[e];
                }
            } else if (slot[k] < 0) {
                continue;                                   // a padding row: its keys and values are stored nowhere
            } else if (c0 < Cq + Ck) {
                const int c = c0 - Cq;
                dst = kdst + (size_t)(c / d) * JANIS_PAGE * d + c % d;
                if (wk != nullptr) {
#pragma unroll
                    for (int e = 0; e < V; e += 4) Vec16<float>::load(wk + c + e, w + e);
#pragma unroll
                    for (int e = 0; e < V; ++e) y[e] = y[e] * ik * w[e];
                }
            } else {
                const int c = c0 - Cq - Ck, g = c / dv;
                dst = vdst + (size_t)g * JANIS_PAGE * dv + c % dv;
                const float iv = inv_s[k * (2 + G) + 2 + g];
#pragma unroll
                for (int e = 0; e < V; ++e) y[e] = y[e] * iv;
            }
            Vec16<T>::store(dst, y);
        }
    }
}

// rows[t]: q (H heads of d + dr) at 0 (or the rows of q_rows, when the queries come from a product of their own), and
// at lat_off the compressed row [c (R) | r (dr)].
// qfull[t, h, R : R + dr] = turn(q[t, h, d : d + dr]); the line's key at the token's position = [norm(c) | turn(r)].
// The turned pairs are neighbours (2p, 2p + 1) or, with `halves`, (p, p + rot/2); features from `rot` on pass as they are.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rotate_store_kernel(const T* __restrict__ rows, int row_elems, int lat_off, const T* __restrict__ q_rows,
                           int q_row_elems, int halves, int H, int d, int dr, int rot, int R,
                           const float* __restrict__ wc, float eps, const float* __restrict__ inv_freq, float amp,
                           const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                           const int* __restrict__ seq_slot, T* __restrict__ qfull, T* __restrict__ kpool,
                           const int* __restrict__ page_table, int table_stride) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    T* kdst = nullptr;
    if (slot >= 0) {
        const int page = page_table[(size_t)slot * table_stride + pos / JANIS_PAGE];
        kdst = kpool + ((size_t)page * JANIS_PAGE + pos % JANIS_PAGE) * (R + dr);
    }
    grid_dependency_wait();
    const T* row = rows + (size_t)t * row_elems;
    const T* qrow = q_rows != nullptr ? q_rows + (size_t)t * q_row_elems : row;
    const T* lat = row + lat_off;
    float ss = 0.f;
    for (int c = tid; c < R; c += nt) {
        const float v = to_float(lat[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)R + eps);
    if (kdst != nullptr)
        for (int c = tid; c < R; c += nt) kdst[c] = from_float<T>(to_float(lat[c]) * inv * wc[c]);
    const int hr = dr >> 1, D = R + dr;
    // unit 0 is the shared key part, units 1 .. H the query heads
    for (int u = tid; u < (H + 1) * hr; u += nt) {
        const int unit = u / hr, p = u % hr;
        float sn = 0.f, cs = 1.f;                             // pairs from rot / 2 on pass as they are
        if (2 * p < rot) {
            sincosf((float)pos * inv_freq[p], &sn, &cs);
            sn *= amp;
            cs *= amp;
        }
        const T* src = unit == 0 ? lat + R : qrow + (size_t)(unit - 1) * (d + dr) + d;
        // where the pair sits: neighbours, or half the turned width apart (the pairs that pass lie behind the turned ones)
        const int ia = !halves ? 2 * p : (2 * p < rot ? p : 2 * p), ib = !halves ? 2 * p + 1 : (2 * p < rot ? p + (rot >> 1) : 2 * p + 1);
        const float a = to_float(src[ia]), b = to_float(src[ib]);
        const float lo = a * cs - b * sn, hi = b * cs + a * sn;
        if (unit == 0) {
            if (kdst != nullptr) {
                kdst[R + ia] = from_float<T>(lo);
                kdst[R + ib] = from_float<T>(hi);
            }
        } else {
            T* dst = qfull + ((size_t)t * H + (unit - 1)) * D + R;
            dst[ia] = from_float<T>(lo);
            dst[ib] = from_float<T>(hi);
        }
    }
}

// Queries and keys that are turned and then divided by their own root mean square, head by head, and values that are
// the keys as they were projected.  rows[t]: q (H heads of d) at 0, k (G heads of d) behind them.  The first `rot`
// features of every head turn by the token's position (pairs (2p, 2p + 1), or (p, p + rot/2) with `halves`; angle
// pos * inv_freq[p]); with unit_norm every head is then divided by sqrt(mean(head^2) + eps).  q is written back in
// place; k goes to the line's keys at the token's position and, when vpool is given, k as projected to its values.
// A CTA per token, a warp per head; the head passes through shared memory as floats.
constexpr int QKN_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(QKN_WARPS * 32)
qk_rotate_norm_store_kernel(T* __restrict__ rows, int row_elems, int H, int G, int d, int rot, int halves,
                            const float* __restrict__ inv_freq, int unit_norm, float eps,
                            const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                            const int* __restrict__ seq_slot, T* __restrict__ kpool, T* __restrict__ vpool,
                            const int* __restrict__ page_table, int table_stride) {
    extern __shared__ float qkn_smem[];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = qkn_smem + (size_t)warp * d;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    size_t kat = 0;
    if (slot >= 0) {
        const int page = page_table[(size_t)slot * table_stride + pos / JANIS_PAGE];
        kat = ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * d;
    }
    grid_dependency_wait();
    T* row = rows + (size_t)t * row_elems;
    const int hr = rot >> 1;
    for (int head = warp; head < H + G; head += QKN_WARPS) {
        const bool is_key = head >= H;
        if (is_key && slot < 0) continue;                    // a padding row's keys are stored nowhere
        T* src = row + (size_t)head * d;
        T* kd = is_key ? kpool + kat + (size_t)(head - H) * JANIS_PAGE * d : nullptr;
        T* vd = is_key && vpool != nullptr ? vpool + kat + (size_t)(head - H) * JANIS_PAGE * d : nullptr;
        float ss = 0.f;
        for (int p = lane; p < hr; p += 32) {
            const int ia = halves ? p : 2 * p, ib = halves ? p + hr : 2 * p + 1;
            float sn, cs;
            sincosf((float)pos * inv_freq[p], &sn, &cs);
            const T ra = src[ia], rb = src[ib];
            const float a = to_float(ra), b = to_float(rb);
            const float lo = a * cs - b * sn, hi = b * cs + a * sn;
            buf[ia] = lo;
            buf[ib] = hi;
            ss = fmaf(lo, lo, ss);
            ss = fmaf(hi, hi, ss);
            if (vd != nullptr) { vd[ia] = ra; vd[ib] = rb; }
        }
        for (int c = rot + lane; c < d; c += 32) {
            const T r = src[c];
            const float v = to_float(r);
            buf[c] = v;
            ss = fmaf(v, v, ss);
            if (vd != nullptr) vd[c] = r;
        }
        ss = warp_sum(ss);
        const float inv = unit_norm ? 1.f / sqrtf(ss / (float)d + eps) : 1.f;
        __syncwarp();
        T* dst = is_key ? kd : src;
        for (int c = lane; c < d; c += 32) dst[c] = from_float<T>(buf[c] * inv);
        __syncwarp();
    }
}

// out[t, h * o_head + o_off + o] = sum_i W[h, o, i] x[t, h * x_head + x_off + i]; a CTA takes 8 tokens of one head and 8
// outputs, a warp an output: lanes stride over i, then a butterfly.
constexpr int HL_TOK = 8, HL_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(HL_WARPS * 32)
head_linear_kernel(const T* __restrict__ x, int x_stride, int x_head, int x_off, const T* __restrict__ w,
                   T* __restrict__ out, int o_stride, int o_head, int o_off, int n_tok, int I, int O) {
    extern __shared__ float hl_smem[];
    const int t0 = blockIdx.x * HL_TOK, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_here = min(HL_TOK, n_tok - t0);
    grid_dependents_launch();
    grid_dependency_wait();
    for (int u = tid; u < HL_TOK * I; u += HL_WARPS * 32) {
        const int tt = u / I, i = u % I;
        hl_smem[u] = tt < n_here ? to_float(x[(size_t)(t0 + tt) * x_stride + (size_t)h * x_head + x_off + i]) : 0.f;
    }
    __syncthreads();
    for (int o = blockIdx.z * HL_WARPS + warp; o < O; o += gridDim.z * HL_WARPS) {
        const T* wr = w + ((size_t)h * O + o) * I;
        float acc[HL_TOK];
#pragma unroll
        for (int tt = 0; tt < HL_TOK; ++tt) acc[tt] = 0.f;
        for (int i = lane; i < I; i += 32) {
            const float wv = to_float(wr[i]);
#pragma unroll
            for (int tt = 0; tt < HL_TOK; ++tt) acc[tt] = fmaf(wv, hl_smem[tt * I + i], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_TOK; ++tt) {
            const float v = warp_sum(acc[tt]);
            if (lane == 0 && tt < n_here)
                out[(size_t)(t0 + tt) * o_stride + (size_t)h * o_head + o_off + o] = from_float<T>(v);
        }
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_qkv_conv_norm_store(const void* rows, int dtype, int row_elems, int T, int H, int G, int d, int dv,
                                           int K, const float* conv_w, float* conv_state, const float* wq,
                                           const float* wk, int v_unit, float eps, const int* tok_pos,
                                           const int* tok_seq, const int* seq_slot, const int* seq_first_row,
                                           const int* seq_start, const int* seq_end, void* q_out, void* kpool,
                                           void* vpool, const int* page_table, int table_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long C = (long long)H * d + (long long)G * (d + dv);
    if (H <= 0 || G <= 0 || d <= 0 || dv <= 0 || row_elems < C) return fail("qkv_conv_norm_store: rows of %d elements do not hold %d + %d heads", row_elems, H, G);
    if (conv_w != nullptr && (K < 1 || K > 16)) return fail("qkv_conv_norm_store: %d taps (1 to 16 are taken)", K);
    if (conv_w != nullptr && K > 1 && conv_state == nullptr) return fail("qkv_conv_norm_store: a filter needs its kept inputs");
    const size_t bytes = ((size_t)C + 2 + G + 32) * sizeof(float);
    if (bytes > 200 * 1024) return fail("qkv_conv_norm_store: a row of %lld channels does not fit shared memory", C);
    // 16 bytes at a time where every head starts on such a border and the taps are few
    const int taps = conv_w != nullptr ? K : 1;
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int V = dtype == JANIS_F32 ? 4 : 8;
    const bool vec = taps <= 4 && d % V == 0 && dv % V == 0 && row_elems % V == 0 && aligned(rows) && aligned(q_out) &&
                     aligned(kpool) && aligned(vpool) && aligned(conv_w) && aligned(conv_state) && aligned(wq) && aligned(wk);
#define JANIS_PREP_VEC(TT, KT, TOK)                                                                                    \
    {                                                                                                                  \
        static size_t most = 0;                                                                                        \
        const size_t vbytes = ((size_t)TOK * (C + 2 + G) + (PREP_THREADS / 32) * 2 * TOK) * sizeof(float);             \
        if (vbytes > most && vbytes > 48 * 1024) {                                                                     \
            cudaError_t e = cudaFuncSetAttribute(qkv_conv_norm_store_vec_kernel<TT, KT, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)vbytes); \
            if (e != cudaSuccess) return fail("qkv_conv_norm_store: shared memory of %zu bytes refused: %s", vbytes, cudaGetErrorString(e)); \
            most = vbytes;                                                                                             \
        }                                                                                                              \
        return launch_kernel("qkv_conv_norm_store", qkv_conv_norm_store_vec_kernel<TT, KT, TOK>,                       \
                             dim3((T + TOK - 1) / TOK), dim3(PREP_THREADS), vbytes, stream, 1, (const TT*)rows,        \
                             row_elems, T, H, G, d, dv, conv_w, conv_state, wq, wk, v_unit, eps, tok_pos, tok_seq,     \
                             seq_slot, seq_first_row, seq_start, seq_end, (TT*)q_out, (TT*)kpool, (TT*)vpool,          \
                             page_table, table_stride);                                                                \
    }
#define JANIS_PREP_VEC_TAPS(TT, TOK)                                                                                   \
    {                                                                                                                  \
        if (taps == 1) JANIS_PREP_VEC(TT, 1, TOK)                                                                      \
        if (taps == 2) JANIS_PREP_VEC(TT, 2, TOK)                                                                      \
        if (taps == 3) JANIS_PREP_VEC(TT, 3, TOK)                                                                      \
        JANIS_PREP_VEC(TT, 4, TOK)                                                                                     \
    }
    // four rows a CTA (or two) where the step has rows enough to fill the GPU so and as many filtered rows fit
    // shared memory twice per SM
    const size_t one_row = (size_t)(C + 2 + G) * sizeof(float);
    const int per_cta = T < PREP_MANY_ROWS ? 1 : 4 * one_row <= 96 * 1024 ? 4 : 2 * one_row <= 96 * 1024 ? 2 : 1;
    if (vec && per_cta == 4 && dtype == JANIS_F32) JANIS_PREP_VEC_TAPS(float, 4)
    if (vec && per_cta == 4 && dtype == JANIS_BF16) JANIS_PREP_VEC_TAPS(bf16, 4)
    if (vec && per_cta == 2 && dtype == JANIS_F32) JANIS_PREP_VEC_TAPS(float, 2)
    if (vec && per_cta == 2 && dtype == JANIS_BF16) JANIS_PREP_VEC_TAPS(bf16, 2)
    if (vec && dtype == JANIS_F32) JANIS_PREP_VEC_TAPS(float, 1)
    if (vec && dtype == JANIS_BF16) JANIS_PREP_VEC_TAPS(bf16, 1)
#undef JANIS_PREP_VEC_TAPS
#undef JANIS_PREP_VEC
#define JANIS_PREP_LAUNCH(TT)                                                                                          \
    {                                                                                                                  \
        static size_t most = 0;                                                                                        \
        if (bytes > most && bytes > 48 * 1024) {                                                                       \
            cudaError_t e = cudaFuncSetAttribute(qkv_conv_norm_store_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); \
            if (e != cudaSuccess) return fail("qkv_conv_norm_store: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e)); \
            most = bytes;                                                                                              \
        }                                                                                                              \
        return launch_kernel("qkv_conv_norm_store", qkv_conv_norm_store_kernel<TT>, dim3(T), dim3(PREP_THREADS), bytes, \
                             stream, 1, (const TT*)rows, row_elems, H, G, d, dv, K, conv_w, conv_state, wq, wk, v_unit, \
                             eps, tok_pos, tok_seq, seq_slot, seq_first_row, seq_start, seq_end, (TT*)q_out, (TT*)kpool, \
                             (TT*)vpool, page_table, table_stride);                                                    \
    }
    if (dtype == JANIS_F32) JANIS_PREP_LAUNCH(float)
    if (dtype == JANIS_BF16) JANIS_PREP_LAUNCH(bf16)
#undef JANIS_PREP_LAUNCH
    return fail("qkv_conv_norm_store: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_latent_rotate_store(const void* rows, int dtype, int row_elems, int lat_off, const void* q_rows,
                                           int q_row_elems, int halves, int T, int H, int d,
                                           int dr, int rot, int R, const float* wc, float eps, const float* inv_freq, float amp,
                                           const int* tok_pos, const int* tok_seq, const int* seq_slot, void* qfull,
                                           void* kpool, const int* page_table, int table_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d < 0 || dr < 0 || (dr & 1) || R <= 0) return fail("latent_rotate_store: sizes %d heads, %d + %d, rank %d", H, d, dr, R);
    if (rot < 0 || (rot & 1) || rot > dr) return fail("latent_rotate_store: %d of %d features turned", rot, dr);
    if (lat_off < (q_rows == nullptr ? H * (d + dr) : 0) || lat_off + R + dr > row_elems || (q_rows != nullptr && q_row_elems < H * (d + dr)))
        return fail("latent_rotate_store: rows of %d elements are too short", row_elems);
    if (dtype == JANIS_F32)
        return launch_kernel("latent_rotate_store", latent_rotate_store_kernel<float>, dim3(T), dim3(128), 0, stream, 1,
                             (const float*)rows, row_elems, lat_off, (const float*)q_rows, q_row_elems, halves, H, d, dr, rot, R, wc, eps, inv_freq, amp, tok_pos, tok_seq,
                             seq_slot, (float*)qfull, (float*)kpool, page_table, table_stride);
    if (dtype == JANIS_BF16)
        return launch_kernel("latent_rotate_store", latent_rotate_store_kernel<bf16>, dim3(T), dim3(128), 0, stream, 1,
                             (const bf16*)rows, row_elems, lat_off, (const bf16*)q_rows, q_row_elems, halves, H, d, dr, rot, R, wc, eps, inv_freq, amp, tok_pos, tok_seq,
                             seq_slot, (bf16*)qfull, (bf16*)kpool, page_table, table_stride);
    return fail("latent_rotate_store: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_qk_rotate_norm_store(void* rows, int dtype, int row_elems, int T, int H, int G, int d, int rot,
                                            int halves, const float* inv_freq, int unit_norm, float eps,
                                            const int* tok_pos, const int* tok_seq, const int* seq_slot, void* kpool,
                                            void* vpool, const int* page_table, int table_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || d <= 0) return fail("qk_rotate_norm_store: sizes %d heads over %d, %d", H, G, d);
    if (rot < 0 || (rot & 1) || rot > d) return fail("qk_rotate_norm_store: %d of %d features turned", rot, d);
    if ((H + G) * d > row_elems) return fail("qk_rotate_norm_store: rows of %d elements are too short", row_elems);
    const size_t smem = (size_t)QKN_WARPS * d * sizeof(float);
    if (smem > 48 * 1024) return fail("qk_rotate_norm_store: heads of %d features do not fit shared memory", d);
    if (dtype == JANIS_F32)
        return launch_kernel("qk_rotate_norm_store", qk_rotate_norm_store_kernel<float>, dim3(T), dim3(QKN_WARPS * 32), smem,
                             stream, 1, (float*)rows, row_elems, H, G, d, rot, halves, inv_freq, unit_norm, eps, tok_pos,
                             tok_seq, seq_slot, (float*)kpool, (float*)vpool, page_table, table_stride);
    if (dtype == JANIS_BF16)
        return launch_kernel("qk_rotate_norm_store", qk_rotate_norm_store_kernel<bf16>, dim3(T), dim3(QKN_WARPS * 32), smem,
                             stream, 1, (bf16*)rows, row_elems, H, G, d, rot, halves, inv_freq, unit_norm, eps, tok_pos,
                             tok_seq, seq_slot, (bf16*)kpool, (bf16*)vpool, page_table, table_stride);
    return fail("qk_rotate_norm_store: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_head_linear(const void* x, int dtype, int x_stride, int x_head, int x_off, const void* w, void* out,
                                   int o_stride, int o_head, int o_off, int T, int H, int I, int O, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || I <= 0 || O <= 0) return fail("head_linear: %d heads, %d -> %d", H, I, O);
    const size_t bytes = (size_t)HL_TOK * I * sizeof(float);
    if (bytes > 48 * 1024) return fail("head_linear: heads of %d inputs do not fit shared memory", I);
    int gz = (O + HL_WARPS - 1) / HL_WARPS;
    if (gz > 65535) gz = 65535;
    if (H > 65535) return fail("head_linear: too many heads (%d)", H);
    const dim3 grid((T + HL_TOK - 1) / HL_TOK, H, gz), block(HL_WARPS * 32);
    if (dtype == JANIS_F32)
        return launch_kernel("head_linear", head_linear_kernel<float>, grid, block, bytes, stream, 1, (const float*)x, x_stride,
                             x_head, x_off, (const float*)w, (float*)out, o_stride, o_head, o_off, T, I, O);
    if (dtype == JANIS_BF16)
        return launch_kernel("head_linear", head_linear_kernel<bf16>, grid, block, bytes, stream, 1, (const bf16*)x, x_stride,
                             x_head, x_off, (const bf16*)w, (bf16*)out, o_stride, o_head, o_off, T, I, O);
    return fail("head_linear: unknown dtype %d", dtype);
}
