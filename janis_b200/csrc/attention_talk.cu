// Attention whose heads talk to each other, before the softmax or after it, over the paged cache.
//
//   raw_g[i, j]   = (q_g[i] . k_kv(g)[j]) * scale            for every query head g
//   s_h[i, j]     = sum_g M[h, g] raw_g[i, j]                (M: heads x heads, optional)
//   p_h[i, j]     = exp(s_h[i, j]) / (sink + sum_j' exp(s_h[i, j']))   over the keys j that i sees
//   o_h[i]        = sum_j p_h[i, j] v_kv(h)[j]
//
// A key j is seen by the query at position i when j <= i and, with a block size B > 0, floor(j / B) ==
// floor(i / B), and, with a window W > 0, i - j < W or j < keep_first (the sequence's first positions stay seen behind the
// window, at their true positions).  sink is 1 (a key of score 0 without a value) or 0.  Keys have `d` features and values `dv`,
// which need not be equal.  Values may be stored rotated by their own position (pairs m, m + dv/2, angle
// j * inv_v[m]); the head's output is then turned back by the query's position.
//
// Options: a cap on the scaled scores, raw <- cap tanh(raw / cap), before anything else; a learnt sink per head
// (sink_vals: exp(sink_h) joins the denominator instead of 1); values that are the first dv features of the cached
// keys (v_stride = d: a line that keeps one vector per position for both); and the heads mixed *after* the
// softmax, p'_h = sum_g M[h, g] softmax(raw_g), which takes two passes over the keys: the first leaves every
// (row, head)'s maximum and denominator (`stats`), the second forms the final weights of all heads for a tile of
// keys, mixes them and adds the values up; nothing is rescaled in it.
//
// Every kernel here reads keys and values from the cache line only, so a step stores first and attends
// afterwards, and a prompt that continues, a decode step and a layer that reads another layer's line are the
// same launch.  Sizes are run-time numbers.  Scores, weights and sums are float whatever is stored.
#include "common.cuh"

#include <math_constants.h>

namespace janis {

// ---------------------------------------------------------------------------
// Rotary encoding of a step's queries and keys (first `rot` features, pairs i, i + rot/2), rotation of its
// values over all dv features when inv_v is given, and the write of keys and values into the paged cache
// line.  A row of the step holds q (H heads of d), then k (G heads of d), then v (G heads of dv); a layer
// that only reads a line has rows of q alone (with_kv == 0).  One CTA per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
qkv_rotate_store_kernel(T* __restrict__ rows, int row_elems, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                        const float* __restrict__ inv_qk, int rot, const float* __restrict__ inv_v, int H, int G, int d,
                        int dv, int with_kv, T* __restrict__ kpool, T* __restrict__ vpool,
                        const int* __restrict__ page_table, int table_stride) {
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    grid_dependents_launch();
    const int pos = tok_pos[t];
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (with_kv) {
        const int slot = seq_slot[tok_seq[t]];
        if (slot >= 0) {
            const int page = page_table[(size_t)slot * table_stride + pos / JANIS_PAGE];
            kdst = kpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * d;
            vdst = vpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * dv;
        }
    }
    grid_dependency_wait();
    T* row = rows + (size_t)t * row_elems;
    const int hq = rot >> 1, n_rot_heads = with_kv ? H + G : H;
    for (int u = tid; u < n_rot_heads * hq; u += nt) {
        const int head = u / hq, i = u % hq;
        float s, c;
        sincosf((float)pos * inv_qk[i], &s, &c);
        T* p = row + (size_t)head * d;
        float lo, hi;
        rotate_pair(to_float(p[i]), to_float(p[i + hq]), s, c, lo, hi);
        const T tl = from_float<T>(lo), th = from_float<T>(hi);
        p[i] = tl;
        p[i + hq] = th;
        if (head >= H && kdst) {
            T* kd = kdst + (size_t)(head - H) * JANIS_PAGE * d;
            kd[i] = tl;
            kd[i + hq] = th;
        }
    }
    if (!with_kv) return;
    if (kdst && rot < d) {
        const int rest = d - rot;
        for (int u = tid; u < G * rest; u += nt) {
            const int g = u / rest, c = rot + u % rest;
            kdst[(size_t)g * JANIS_PAGE * d + c] = row[(size_t)(H + g) * d + c];
        }
    }
    T* vrow = row + (size_t)(H + G) * d;
    if (inv_v != nullptr) {
        const int hv = dv >> 1;
        for (int u = tid; u < G * hv; u += nt) {
            const int g = u / hv, m = u % hv;
            float s, c;
            sincosf((float)pos * inv_v[m], &s, &c);
            T* p = vrow + (size_t)g * dv;
            float lo, hi;
            rotate_pair(to_float(p[m]), to_float(p[m + hv]), s, c, lo, hi);
            const T tl = from_float<T>(lo), th = from_float<T>(hi);
            p[m] = tl;
            p[m + hv] = th;
            if (vdst) {
                T* vd = vdst + (size_t)g * JANIS_PAGE * dv;
                vd[m] = tl;
                vd[m + hv] = th;
            }
        }
    } else if (vdst) {
        for (int u = tid; u < G * dv; u += nt) vdst[(size_t)(u / dv) * JANIS_PAGE * dv + u % dv] = vrow[u];
    }
}

// ---------------------------------------------------------------------------
// The plain kernel: one CTA per query token, all heads together, tiles of up to 32 keys staged in shared
// memory as floats.  It is the 32-bit path, and the bfloat16 path of sizes the tensor-core kernel leaves out.
// Sums run in an order that depends on the query's position and the model's sizes alone.
// ---------------------------------------------------------------------------
struct TalkShape {
    int H, G, d, dv;
    int block;          // keys are seen within blocks of this many positions (0: all earlier keys)
    int sink;           // 1: one is added to the softmax's denominator
    int window;         // keys are seen among the query's last `window` positions (0: no such limit)
    int keep_first;     // with a window: the sequence's first `keep_first` positions stay seen behind it
    int kt;             // keys per tile (<= 32)
    float scale;
    float cap;          // > 0: raw <- cap tanh(raw / cap)
    int mode;           // 0: one pass (heads mixed before the softmax, if at all); 1: maxima and denominators only, into
                        // `stats`; 2: the weights from `stats`, mixed over the heads after the softmax, times the values
    int v_stride;       // elements between the value rows of neighbouring positions (dv; d when values live in the keys)
};

__host__ __device__ inline size_t talk_plain_smem_floats(int H, int G, int d, int dv, int kt) {
    return (size_t)H * d + (size_t)H * H + (size_t)kt * (G * d + 1) + (size_t)kt * G * dv + 2 * (size_t)H * kt +
           (size_t)H * dv + 5 * (size_t)H;
}

template <typename T>
__global__ void __launch_bounds__(256)
talk_attention_plain_kernel(const T* __restrict__ q_rows, int q_row_elems, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                            const T* __restrict__ kpool, const T* __restrict__ vpool,
                            const int* __restrict__ page_table, int table_stride, const float* __restrict__ talk,
                            const float* __restrict__ inv_v, T* __restrict__ out, const float* __restrict__ sink_vals,
                            float* __restrict__ stats, TalkShape sh) {
    extern __shared__ float smem[];
    const int H = sh.H, G = sh.G, d = sh.d, dv = sh.dv, KT = sh.kt, rep = H / G;
    const int kstride = G * d + 1;
    float* q_s = smem;
    float* talk_s = q_s + (size_t)H * d;
    float* k_s = talk_s + (size_t)H * H;
    float* v_s = k_s + (size_t)KT * kstride;
    float* raw_s = v_s + (size_t)KT * G * dv;
    float* p_s = raw_s + (size_t)H * KT;
    float* o_s = p_s + (size_t)H * KT;
    float* m_s = o_s + (size_t)H * dv;
    float* l_s = m_s + H;
    float* corr_s = l_s + H;
    float* fm_s = corr_s + H;                         // mode 2: every head's final maximum and 1 / denominator
    float* fl_s = fm_s + H;
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    if (talk != nullptr)
        for (int u = tid; u < H * H; u += nt) talk_s[u] = talk[u];
    grid_dependency_wait();
    T* o_row = out + (size_t)t * H * dv;
    if (slot < 0) {                                   // a padding row: written, never read
        if (sh.mode == 1) {
            for (int u = tid; u < 2 * H; u += nt) stats[(size_t)t * 2 * H + u] = 0.f;
            return;
        }
        for (int u = tid; u < H * dv; u += nt) o_row[u] = from_float<T>(0.f);
        return;
    }
    const T* q = q_rows + (size_t)t * q_row_elems;
    for (int u = tid; u < H * d; u += nt) q_s[u] = to_float(q[u]);
    for (int u = tid; u < H * dv; u += nt) o_s[u] = 0.f;
    for (int u = tid; u < H; u += nt) {
        m_s[u] = sh.sink ? (sink_vals != nullptr ? sink_vals[u] : 0.f) : -CUDART_INF_F;
        l_s[u] = sh.sink ? 1.f : 0.f;
        if (sh.mode == 2) {
            const float L = stats[(size_t)t * 2 * H + 2 * u + 1];
            fm_s[u] = stats[(size_t)t * 2 * H + 2 * u];
            fl_s[u] = L > 0.f ? 1.f / L : 0.f;
            l_s[u] = 1.f;                             // the weights arrive normalised: nothing is divided at the end
            corr_s[u] = 1.f;
        }
    }
    int first = sh.block > 0 ? (pos / sh.block) * sh.block : 0;
    if (sh.window > 0) first = max(first, pos - sh.window + 1);
    // the keys a row sees, counted through: the kept first positions that lie before the window, then first .. pos
    const int kept = sh.window > 0 ? min(sh.keep_first, first) : 0, n_keys = kept + pos - first + 1;
    const int* table = page_table + (size_t)slot * table_stride;
    for (int j0 = 0; j0 < n_keys; j0 += KT) {
        const int kt = min(KT, n_keys - j0);
        __syncthreads();                              // the tile before has been used; q_s and o_s are in place
        for (int u = tid; u < kt * G * d; u += nt) {
            const int jj = u / (G * d), r = u % (G * d), g = r / d, c = r % d, j = j0 + jj < kept ? j0 + jj : first + j0 + jj - kept;
            const size_t at = (((size_t)table[j / JANIS_PAGE] * G + g) * JANIS_PAGE + j % JANIS_PAGE) * d + c;
            k_s[(size_t)jj * kstride + r] = to_float(kpool[at]);
        }
        if (sh.mode != 1)
            for (int u = tid; u < kt * G * dv; u += nt) {
                const int jj = u / (G * dv), r = u % (G * dv), g = r / dv, c = r % dv, j = j0 + jj < kept ? j0 + jj : first + j0 + jj - kept;
                const size_t at = (((size_t)table[j / JANIS_PAGE] * G + g) * JANIS_PAGE + j % JANIS_PAGE) * sh.v_stride + c;
                v_s[(size_t)jj * G * dv + r] = to_float(vpool[at]);
            }
        __syncthreads();
        for (int u = tid; u < H * KT; u += nt) {
            const int g = u / KT, jj = u % KT;
            float acc = 0.f;
            if (jj < kt) {
                const float* qq = q_s + (size_t)g * d;
                const float* kk = k_s + (size_t)jj * kstride + (size_t)(g / rep) * d;
                for (int c = 0; c < d; ++c) acc = fmaf(qq[c], kk[c], acc);
            }
            acc *= sh.scale;
            if (sh.cap > 0.f) acc = sh.cap * tanhf(acc / sh.cap);
            if (sh.mode == 2) acc = jj < kt ? expf(acc - fm_s[g]) * fl_s[g] : 0.f;     // the head's final weight of this key
            raw_s[u] = acc;
        }
        __syncthreads();
        if (sh.mode == 2) {
            // the heads' weights mixed; no maximum, no correction
            for (int u = tid; u < H * KT; u += nt) {
                const int h = u / KT, jj = u % KT;
                float w = raw_s[u];
                if (talk != nullptr) {
                    w = 0.f;
                    for (int g = 0; g < H; ++g) w = fmaf(talk_s[h * H + g], raw_s[g * KT + jj], w);
                }
                p_s[u] = w;
            }
        }
        for (int h = warp; h < H && sh.mode != 2; h += nwarp) {
            float s = -CUDART_INF_F;
            if (lane < kt) {
                if (talk != nullptr && sh.mode == 0) {
                    s = 0.f;
                    for (int g = 0; g < H; ++g) s = fmaf(talk_s[h * H + g], raw_s[g * KT + lane], s);
                } else {
                    s = raw_s[h * KT + lane];         // (mode 1: the head's own scores; the mixing comes after the softmax)
                }
            }
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float p = lane < kt ? expf(s - m_new) : 0.f;
            const float sum = warp_sum(p);
            const float corr = m_old == -CUDART_INF_F ? 0.f : expf(m_old - m_new);
            __syncwarp();
            if (lane == 0) {
                l_s[h] = l_s[h] * corr + sum;
                m_s[h] = m_new;
                corr_s[h] = corr;
            }
            if (lane < KT) p_s[h * KT + lane] = p;
        }
        __syncthreads();
        if (sh.mode == 1) continue;
        for (int u = tid; u < H * dv; u += nt) {
            const int h = u / dv, c = u % dv;
            const float* vv = v_s + (size_t)(h / rep) * dv + c;
            const float* pp = p_s + h * KT;
            float acc = o_s[u] * corr_s[h];
            for (int jj = 0; jj < kt; ++jj) acc = fmaf(pp[jj], vv[(size_t)jj * G * dv], acc);
            o_s[u] = acc;
        }
    }
    __syncthreads();
    if (sh.mode == 1) {
        for (int u = tid; u < H; u += nt) {
            stats[(size_t)t * 2 * H + 2 * u] = m_s[u];
            stats[(size_t)t * 2 * H + 2 * u + 1] = l_s[u];
        }
        return;
    }
    if (inv_v != nullptr) {
        const int hv = dv >> 1;
        for (int u = tid; u < H * hv; u += nt) {
            const int h = u / hv, m = u % hv;
            const float inv_l = 1.f / l_s[h];
            float s, c;
            sincosf((float)pos * inv_v[m], &s, &c);
            float lo, hi;
            rotate_pair(o_s[h * dv + m] * inv_l, o_s[h * dv + m + hv] * inv_l, -s, c, lo, hi);
            o_row[h * dv + m] = from_float<T>(lo);
            o_row[h * dv + m + hv] = from_float<T>(hi);
        }
    } else {
        for (int u = tid; u < H * dv; u += nt) o_row[u] = from_float<T>(o_s[u] / l_s[u / dv]);
    }
}

// ---------------------------------------------------------------------------
// The tensor-core kernel (bfloat16, d a multiple of 16, dv a multiple of 8, up to 32 heads).
//
// A CTA of 16 warps owns up to QR (16 or 8) consecutive rows of the packed step, all heads together, since every
// head's weights need every head's scores.  Rows of one sequence form a run; a run's keys (from the first row's
// block start to the last row's position) come in tiles of BN keys.  Per tile, three phases with the scores
// passing through shared memory as floats:
//   1. raw_g = Q_g K^T * scale for every head (mma.sync m16n8k16, operands by ldmatrix; items (head, 8 keys)
//      dealt to the warps);
//   2. a thread per (row, key) mixes the heads' scores in float registers and applies the mask; a warp per (head,
//      row) then does the online softmax (maximum, exponentials, sum) and leaves P as bfloat16;
//   3. O_h = O_h * corr + P_h V (mma.sync; V through ldmatrix.trans; items (head, 8 value columns) dealt to the
//      warps), the accumulators living in shared memory as floats so that all sizes are run-time numbers.
// Keys and values of a tile take turns in one buffer.  With QR = 8 the upper half of every 16-row operand repeats
// the lower one and is dropped: big heads fit shared memory that way.  A decode step runs one row a CTA and keeps that
// row alone (QR = 1: every row of the 16-row operands repeats it).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

constexpr int TALK_MMA_WARPS = 16, TALK_MMA_THREADS = TALK_MMA_WARPS * 32;

struct TalkMmaShape {
    int H, G, d, dv, block, sink;
    int window;         // keys are seen among the query's last `window` positions (0: no such limit)
    int keep_first;     // with a window: the sequence's first `keep_first` positions stay seen behind it
    int qr;             // rows of the operands kept (16 or 8; 1 in a decode step, whose CTAs own one row each)
    int rows;           // rows of the step a CTA owns (qr, or 1 in a decode step)
    int bn;             // keys per tile (16, 32, 64)
    int chunk;          // keys per CTA of a decode step whose rows are cut over grid.y CTAs (0: a row's keys in one CTA)
    int hg;             // groups the heads are cut into: a CTA forms the scores of all heads and the weights and sums of
                        // its own group (1: all heads in one CTA; more where all heads' sums do not fit shared memory)
    float scale;
    float cap;          // > 0: raw <- cap tanh(raw / cap)
    int mode;           // as TalkShape::mode: 0 one pass; 1 maxima and denominators only; 2 final weights mixed after the softmax
    int v_in_keys;      // the values are the first dv features of the keys: the tile of keys serves as the tile of values
};

struct TalkMmaLayout {
    size_t q, kv, raw, p, o, m, l, corr, talk, fin, meta, total;
    int qs, kvs, rs, ps, os;       // row strides in elements
};

__host__ __device__ inline TalkMmaLayout talk_mma_layout(int H, int G, int d, int dv, int qr, int bn, int hp) {
    TalkMmaLayout L;
    L.qs = d + 8; L.kvs = (d > dv ? d : dv) + 8; L.rs = bn + 4; L.ps = bn + 8; L.os = dv + 4;
    size_t at = 0;
    L.q = at;    at += (size_t)H * qr * L.qs * 2;
    L.kv = at;   at += (size_t)G * bn * L.kvs * 2;
    L.p = at;    at += (size_t)hp * qr * L.ps * 2;
    at = (at + 15) & ~(size_t)15;
    L.raw = at;  at += (size_t)H * qr * L.rs * 4;
    L.o = at;    at += (size_t)hp * qr * L.os * 4;
    L.m = at;    at += (size_t)hp * qr * 4;
    L.l = at;    at += (size_t)hp * qr * 4;
    L.corr = at; at += (size_t)hp * qr * 4;
    L.talk = at; at += (size_t)H * H * 4;
    L.fin = at;  at += (size_t)2 * H * qr * 4;          // mode 2: every (head, row)'s final maximum and 1 / denominator
    L.meta = at; at += (3 * 16 + 2 * 64) * 4;
    L.total = at;
    return L;
}

template <int HMAX>
__global__ void __launch_bounds__(TALK_MMA_THREADS)
talk_attention_mma_kernel(const bf16* __restrict__ q_rows, int q_row_elems, const int* __restrict__ tok_pos,
                          const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                          const bf16* __restrict__ kpool, const bf16* __restrict__ vpool,
                          const int* __restrict__ page_table, int table_stride, const float* __restrict__ talk,
                          const float* __restrict__ inv_v, bf16* __restrict__ out, float* __restrict__ partial,
                          const float* __restrict__ sink_vals, float* __restrict__ stats, int n_tok, TalkMmaShape sh) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = sh.H, G = sh.G, d = sh.d, dv = sh.dv, QR = sh.qr, BN = sh.bn, rep = H / G;
    const int HP = H / sh.hg, h0 = ((int)blockIdx.y % sh.hg) * HP;       // this CTA's heads: h0 .. h0 + HP - 1
    const TalkMmaLayout L = talk_mma_layout(H, G, d, dv, QR, BN, HP);
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw + L.q);
    bf16* kv_s = reinterpret_cast<bf16*>(smem_raw + L.kv);
    bf16* p_s = reinterpret_cast<bf16*>(smem_raw + L.p);
    float* raw_s = reinterpret_cast<float*>(smem_raw + L.raw);
    float* o_s = reinterpret_cast<float*>(smem_raw + L.o);
    float* m_s = reinterpret_cast<float*>(smem_raw + L.m);
    float* l_s = reinterpret_cast<float*>(smem_raw + L.l);
    float* corr_s = reinterpret_cast<float*>(smem_raw + L.corr);
    float* talk_s = reinterpret_cast<float*>(smem_raw + L.talk);
    float* fm_s = reinterpret_cast<float*>(smem_raw + L.fin);
    float* fl_s = fm_s + (size_t)H * QR;
    int* pos_s = reinterpret_cast<int*>(smem_raw + L.meta);
    int* seq_s = pos_s + 16;
    int* slot_s = pos_s + 32;
    int* base_s = pos_s + 48;                  // where each key of the tile starts in the pools (in rows), -1 beyond the last
    int* kpos_s = pos_s + 112;                 // each key's position in its sequence
    const bool split = sh.chunk > 0;           // the CTA leaves a partial result; the sink joins at the merge
    const int bn_log2 = BN == 64 ? 6 : (BN == 32 ? 5 : 4);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the last rows of a prompt see the most keys: they start first
    const int r0 = (int)(gridDim.x - 1 - blockIdx.x) * sh.rows, n_rows = min(sh.rows, n_tok - r0);
    grid_dependents_launch();
    if (tid < 16) {
        const bool in = tid < n_rows;
        const int sq = in ? tok_seq[r0 + tid] : -1;
        pos_s[tid] = in ? tok_pos[r0 + tid] : 0;
        seq_s[tid] = sq;
        slot_s[tid] = in ? seq_slot[sq] : -1;
    }
    if (talk != nullptr)
        for (int u = tid; u < H * H; u += TALK_MMA_THREADS) talk_s[u] = talk[u];
    for (int u = tid; u < HP * QR * L.os; u += TALK_MMA_THREADS) o_s[u] = 0.f;
    for (int u = tid; u < HP * QR; u += TALK_MMA_THREADS) {
        const bool with_sink = sh.sink && !split && sh.mode != 2;
        m_s[u] = with_sink ? (sink_vals != nullptr ? sink_vals[h0 + u / QR] : 0.f) : -CUDART_INF_F;
        l_s[u] = with_sink || sh.mode == 2 ? 1.f : 0.f;      // (mode 2: the weights arrive normalised)
        corr_s[u] = 1.f;
    }
    grid_dependency_wait();
    if (sh.mode == 2)
        for (int u = tid; u < H * QR; u += TALK_MMA_THREADS) {
            const int h = u / QR, r = u & (QR - 1);
            float M = 0.f, inv = 0.f;
            if (r < n_rows) {
                const float Lr = stats[(size_t)(r0 + r) * 2 * H + 2 * h + 1];
                M = stats[(size_t)(r0 + r) * 2 * H + 2 * h];
                inv = Lr > 0.f ? 1.f / Lr : 0.f;
            }
            fm_s[u] = M;
            fl_s[u] = inv;
        }
    // queries: a warp per (head, row), a lane per 16 bytes; rows beyond the step's end are zero
    for (int hr = warp; hr < H * QR; hr += TALK_MMA_WARPS) {
        const int h = hr / QR, r = hr & (QR - 1);
        const bf16* src = q_rows + (size_t)(r0 + (r < n_rows ? r : 0)) * q_row_elems + (size_t)h * d;
        bf16* dst = q_s + (size_t)hr * L.qs;
        for (int c8 = lane; c8 < d / 8; c8 += 32)
            *reinterpret_cast<uint4*>(dst + c8 * 8) = r < n_rows ? *reinterpret_cast<const uint4*>(src + c8 * 8) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    int a = 0;
    while (a < n_rows) {
        int b = a + 1;
        while (b < n_rows && seq_s[b] == seq_s[a]) ++b;
        const int slot = slot_s[a];
        if (slot >= 0) {
            int first = sh.block > 0 ? (pos_s[a] / sh.block) * sh.block : 0, last = pos_s[b - 1];
            if (sh.window > 0) first = max(first, pos_s[a] - sh.window + 1);       // the run's first row reaches back farthest
            // the keys the run sees, counted through: the kept first positions that lie before the window, then
            // first .. last; a decode row's chunks cut this count
            const int kept = sh.window > 0 ? min(sh.keep_first, first) : 0;
            int n_first = 0, n_last = kept + last - first;
            if (split) {
                n_first = ((int)blockIdx.y / sh.hg) * sh.chunk;
                n_last = min(n_last, n_first + sh.chunk - 1);
            }
            const int* table = page_table + (size_t)slot * table_stride;
            for (int j0 = n_first; j0 <= n_last; j0 += BN) {
                // ---- keys of the tile
                if (tid < BN) {
                    const int n = j0 + tid, j = n < kept ? n : first + n - kept;
                    base_s[tid] = n <= n_last ? (table[j / JANIS_PAGE] * G) * JANIS_PAGE + j % JANIS_PAGE : -1;
                    kpos_s[tid] = j;
                }
                __syncthreads();
                // (a warp per row of the tile, a lane per 16 bytes: no divisions in the addresses)
                for (int row = warp; row < G * BN; row += TALK_MMA_WARPS) {
                    const int g = row >> bn_log2, jj = row & (BN - 1), at = base_s[jj];
                    bf16* dst = kv_s + (size_t)row * L.kvs;
                    const bf16* src = kpool + ((size_t)(at < 0 ? 0 : at) + (size_t)g * JANIS_PAGE) * d;
                    for (int c8 = lane; c8 < d / 8; c8 += 32) {
                        if (at >= 0) cp_async16(smem_u32(dst + c8 * 8), src + c8 * 8);
                        else *reinterpret_cast<uint4*>(dst + c8 * 8) = make_uint4(0, 0, 0, 0);
                    }
                }
                cp_async_wait_all();
                __syncthreads();
                // ---- 1: raw scores of every head; a warp takes a head and up to four tiles of 8 keys, which share
                //         the queries' fragments and run as four independent chains
                {
                    const int nts = BN / 8;
                    int tg = 4;                               // tiles a unit: fewer where the warps would outnumber the units
                    while (tg > 1 && (talk == nullptr || sh.mode == 1 ? HP : H) * ((nts + tg - 1) / tg) < TALK_MMA_WARPS) tg >>= 1;
                    const int groups = (nts + tg - 1) / tg;
                    // (where nothing mixes the heads' scores, a CTA forms those of its own heads alone)
                    const bool own_only = talk == nullptr || sh.mode == 1;
                    const int g_first = own_only ? h0 : 0, g_count = own_only ? HP : H;
                    for (int unit = warp; unit < g_count * groups; unit += TALK_MMA_WARPS) {
                        const int g = g_first + unit / groups, nt0 = (unit % groups) * tg, n_here = min(tg, nts - nt0), kvh = g / rep;
                        float acc[4][4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                        const uint32_t a_base = smem_u32(q_s + ((size_t)g * QR + ((lane & 15) & (QR - 1))) * L.qs + (lane >> 4) * 8);
                        const uint32_t b_base = smem_u32(kv_s + ((size_t)kvh * BN + nt0 * 8 + (lane & 7)) * L.kvs + ((lane >> 3) & 1) * 8);
                        const uint32_t b_step = (uint32_t)(8 * L.kvs * 2);
                        for (int kk = 0; kk < d / 16; ++kk) {
                            uint32_t af[4];
                            ldsm_x4(af, a_base + kk * 32);
#pragma unroll
                            for (int t = 0; t < 4; ++t)
                                if (t < n_here) {
                                    uint32_t bfr[2];
                                    ldsm_x2(bfr, b_base + t * b_step + kk * 32);
                                    mma_bf16(acc[t], af, bfr);
                                }
                        }
                        const int r = lane >> 2;
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if (t < n_here) {
                                if (r >= QR) continue;        // (one row kept: the other rows of the operand repeat it)
                                float* dst = raw_s + ((size_t)g * QR + r) * L.rs + (nt0 + t) * 8 + (lane & 3) * 2;
                                float z[4] = {acc[t][0] * sh.scale, acc[t][1] * sh.scale, acc[t][2] * sh.scale, acc[t][3] * sh.scale};
                                if (sh.cap > 0.f) {
#pragma unroll
                                    for (int e = 0; e < 4; ++e) z[e] = sh.cap * tanhf(z[e] / sh.cap);
                                }
                                dst[0] = z[0];
                                dst[1] = z[1];
                                if (QR == 16) {
                                    dst[8 * L.rs] = z[2];
                                    dst[8 * L.rs + 1] = z[3];
                                }
                            }
                    }
                }
                __syncthreads();
                // ---- 2a: the heads' scores mixed, the mask
                for (int pair = tid; pair < QR * BN; pair += TALK_MMA_THREADS) {
                    const int r = pair >> bn_log2, c = pair & (BN - 1), j = kpos_s[c];
                    bool seen = r >= a && r < b && j <= pos_s[r] && base_s[c] >= 0;
                    if (seen && sh.block > 0) seen = j >= (pos_s[r] / sh.block) * sh.block;
                    if (seen && sh.window > 0) seen = j > pos_s[r] - sh.window || j < sh.keep_first;
                    float* at = raw_s + (size_t)r * L.rs + c;
                    const size_t hs = (size_t)QR * L.rs;
                    if (sh.mode == 2) {
                        // every head's final weight of this key, mixed over the heads; P is written here
                        float w[HMAX];
#pragma unroll
                        for (int g = 0; g < HMAX; ++g)
                            w[g] = g < H && seen ? expf(at[g * hs] - fm_s[g * QR + r]) * fl_s[g * QR + r] : 0.f;
                        for (int h = h0; h < h0 + HP; ++h) {
                            float s = w[0];
                            if (talk != nullptr) {
                                const float* tr = talk_s + h * H;
                                s = 0.f;
#pragma unroll
                                for (int g = 0; g < HMAX; ++g)
                                    if (g < H) s = fmaf(tr[g], w[g], s);
                            } else {
#pragma unroll
                                for (int g = 0; g < HMAX; ++g)
                                    if (g == h) s = w[g];
                            }
                            p_s[((size_t)(h - h0) * QR + r) * L.ps + c] = __float2bfloat16_rn(s);
                        }
                    } else if (!seen) {
                        for (int h = h0; h < h0 + HP; ++h) at[h * hs] = -CUDART_INF_F;
                    } else if (talk != nullptr && sh.mode == 0) {
                        float raw[HMAX];
#pragma unroll
                        for (int g = 0; g < HMAX; ++g) raw[g] = g < H ? at[g * hs] : 0.f;
                        for (int h = h0; h < h0 + HP; ++h) {
                            const float* tr = talk_s + h * H;
                            float s = 0.f;
#pragma unroll
                            for (int g = 0; g < HMAX; ++g)
                                if (g < H) s = fmaf(tr[g], raw[g], s);
                            at[h * hs] = s;
                        }
                    }
                }
                __syncthreads();
                // ---- 2b: online softmax of every (head, row); P as bfloat16
                for (int u = warp; u < HP * QR && sh.mode != 2; u += TALK_MMA_WARPS) {
                    const float* src = raw_s + ((size_t)h0 * QR + u) * L.rs;
                    const float s0 = lane < BN ? src[lane] : -CUDART_INF_F;
                    const float s1 = lane + 32 < BN ? src[lane + 32] : -CUDART_INF_F;
                    const float m_old = m_s[u];
                    const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
                    float p0 = 0.f, p1 = 0.f, corr = 1.f;
                    if (m_new != -CUDART_INF_F) {
                        p0 = expf(s0 - m_new);
                        p1 = expf(s1 - m_new);
                        corr = m_old == -CUDART_INF_F ? 0.f : expf(m_old - m_new);
                    }
                    const float sum = warp_sum(p0 + p1);
                    __syncwarp();
                    if (lane == 0) {
                        m_s[u] = m_new;
                        l_s[u] = l_s[u] * corr + sum;
                        corr_s[u] = corr;
                    }
                    bf16* dst = p_s + (size_t)u * L.ps;
                    if (lane < BN) dst[lane] = __float2bfloat16_rn(p0);
                    if (lane + 32 < BN) dst[lane + 32] = __float2bfloat16_rn(p1);
                }
                __syncthreads();
                if (sh.mode == 1) continue;                  // (the barrier at the top of the next tile's load orders the reuse)
                // ---- values of the tile, into the keys' place (values that lie in the keys are there already)
                for (int row = warp; row < G * BN && !sh.v_in_keys; row += TALK_MMA_WARPS) {
                    const int g = row >> bn_log2, jj = row & (BN - 1), at = base_s[jj];
                    bf16* dst = kv_s + (size_t)row * L.kvs;
                    const bf16* src = vpool + ((size_t)(at < 0 ? 0 : at) + (size_t)g * JANIS_PAGE) * dv;
                    for (int c8 = lane; c8 < dv / 8; c8 += 32) {
                        if (at >= 0) cp_async16(smem_u32(dst + c8 * 8), src + c8 * 8);
                        else *reinterpret_cast<uint4*>(dst + c8 * 8) = make_uint4(0, 0, 0, 0);     // 0 x NaN is NaN
                    }
                }
                cp_async_wait_all();
                __syncthreads();
                // ---- 3: O = O corr + P V; a warp takes a head and up to four tiles of 8 value columns, which share
                //         P's fragments and run as four independent chains
                {
                    const int nts = dv / 8, groups = (nts + 3) / 4;
                    for (int unit = warp; unit < HP * groups; unit += TALK_MMA_WARPS) {
                        const int h = unit / groups, nt0 = (unit % groups) * 4, n_here = min(4, nts - nt0), kvh = (h0 + h) / rep;
                        const bool mine = (lane >> 2) < QR;            // this lane's row of the sums is kept
                        const int r = mine ? lane >> 2 : 0;
                        const float c_lo = corr_s[h * QR + r], c_hi = QR == 16 ? corr_s[h * QR + r + 8] : 0.f;
                        float* op = o_s + ((size_t)h * QR + r) * L.os + nt0 * 8 + (lane & 3) * 2;
                        float acc[4][4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                            if (t < n_here && mine) {
                                acc[t][0] = op[t * 8] * c_lo;
                                acc[t][1] = op[t * 8 + 1] * c_lo;
                                if (QR == 16) {
                                    acc[t][2] = op[8 * L.os + t * 8] * c_hi;
                                    acc[t][3] = op[8 * L.os + t * 8 + 1] * c_hi;
                                }
                            }
                        }
                        const uint32_t a_base = smem_u32(p_s + ((size_t)h * QR + ((lane & 15) & (QR - 1))) * L.ps + (lane >> 4) * 8);
                        const uint32_t b_base = smem_u32(kv_s + ((size_t)kvh * BN + (lane & 15)) * L.kvs + nt0 * 8);
                        for (int kk = 0; kk < BN / 16; ++kk) {
                            uint32_t af[4];
                            ldsm_x4(af, a_base + kk * 32);
#pragma unroll
                            for (int t = 0; t < 4; ++t)
                                if (t < n_here) {
                                    uint32_t bfr[2];
                                    ldsm_x2_trans(bfr, b_base + (uint32_t)(kk * 16 * L.kvs * 2) + t * 16);
                                    mma_bf16(acc[t], af, bfr);
                                }
                        }
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if (t < n_here && mine) {
                                op[t * 8] = acc[t][0];
                                op[t * 8 + 1] = acc[t][1];
                                if (QR == 16) {
                                    op[8 * L.os + t * 8] = acc[t][2];
                                    op[8 * L.os + t * 8 + 1] = acc[t][3];
                                }
                            }
                    }
                }
                __syncthreads();
            }
        }
        a = b;
    }
    __syncthreads();
    if (sh.mode == 1 && !split) {
        // every (row, head)'s maximum and denominator, for the pass that forms the weights
        for (int u = tid; u < n_rows * HP; u += TALK_MMA_THREADS) {
            const int h = u % HP, r = u / HP;
            const bool live = slot_s[r] >= 0;
            float* dst = stats + (size_t)(r0 + r) * 2 * H + 2 * (h0 + h);
            dst[0] = live ? m_s[h * QR + r] : 0.f;
            dst[1] = live ? l_s[h * QR + r] : 0.f;
        }
        return;
    }
    if (split) {
        // the chunk's share of row r0: per head the unnormalised sums, then the maximum and the denominator.  (Weights
        // that are final already, mode 2, add up as they are: maximum 0, and the first chunk alone brings the 1 that
        // the sums are divided by.)
        const int chunk_id = (int)blockIdx.y / sh.hg;
        float* dst = partial + ((size_t)r0 * (gridDim.y / sh.hg) + chunk_id) * H * (dv + 2) + (size_t)h0 * (dv + 2);
        for (int u = tid; u < HP * (dv + 2); u += TALK_MMA_THREADS) {
            const int h = u / (dv + 2), c = u % (dv + 2);
            float x;
            if (c < dv) x = sh.mode == 1 ? 0.f : o_s[(size_t)h * QR * L.os + c];
            else if (sh.mode == 2) x = c == dv ? 0.f : (chunk_id == 0 ? 1.f : 0.f);
            else x = c == dv ? m_s[h * QR] : l_s[h * QR];
            dst[u] = x;
        }
        return;
    }
    // ---- the way out: divide, turn back by the row's position, round
    const int hv = dv >> 1;
    for (int u = tid; u < n_rows * HP * hv; u += TALK_MMA_THREADS) {
        const int m = u % hv, h = (u / hv) % HP, r = u / (hv * HP);
        bf16* o_row = out + (size_t)(r0 + r) * H * dv + (size_t)(h0 + h) * dv;
        float lo = 0.f, hi = 0.f;
        if (slot_s[r] >= 0) {
            const float inv_l = 1.f / l_s[h * QR + r];
            const float* src = o_s + ((size_t)h * QR + r) * L.os;
            if (inv_v != nullptr) {
                float s, c;
                sincosf((float)pos_s[r] * inv_v[m], &s, &c);
                rotate_pair(src[m] * inv_l, src[m + hv] * inv_l, -s, c, lo, hi);
            } else {
                lo = src[m] * inv_l;
                hi = src[m + hv] * inv_l;
            }
        }
        o_row[m] = __float2bfloat16_rn(lo);
        o_row[m + hv] = __float2bfloat16_rn(hi);
    }
}

// The chunks of a decode row put together, in ascending order: per head the maximum over the chunks (and the
// sink's 0), the weights exp(m_c - M), the denominators and sums added, divided, turned back, rounded.
__global__ void __launch_bounds__(128)
talk_attention_merge_kernel(const float* __restrict__ partial, int n_chunks, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                            const float* __restrict__ inv_v, bf16* __restrict__ out, int H, int dv, int sink,
                            const float* __restrict__ sink_vals) {
    const int t = blockIdx.x, tid = threadIdx.x;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    grid_dependency_wait();
    const int hv = dv >> 1;
    const float* base = partial + (size_t)t * n_chunks * H * (dv + 2);
    for (int u = tid; u < H * hv; u += blockDim.x) {
        const int h = u / hv, m = u % hv;
        float lo = 0.f, hi = 0.f;
        if (slot >= 0) {
            const float* ph = base + (size_t)h * (dv + 2);
            const size_t cs = (size_t)H * (dv + 2);
            const float z = sink_vals != nullptr ? sink_vals[h] : 0.f;
            float M = sink ? z : -CUDART_INF_F;
            for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, ph[c * cs + dv]);
            float Lsum = sink ? expf(z - M) : 0.f, a0 = 0.f, a1 = 0.f;
            for (int c = 0; c < n_chunks; ++c) {
                const float mc = ph[c * cs + dv];
                if (mc == -CUDART_INF_F) continue;
                const float w = expf(mc - M);
                Lsum = fmaf(w, ph[c * cs + dv + 1], Lsum);
                a0 = fmaf(w, ph[c * cs + m], a0);
                a1 = fmaf(w, ph[c * cs + m + hv], a1);
            }
            const float inv_l = 1.f / Lsum;
            if (inv_v != nullptr) {
                float s, c;
                sincosf((float)pos * inv_v[m], &s, &c);
                rotate_pair(a0 * inv_l, a1 * inv_l, -s, c, lo, hi);
            } else {
                lo = a0 * inv_l;
                hi = a1 * inv_l;
            }
        }
        bf16* o_row = out + (size_t)t * H * dv + (size_t)h * dv;
        o_row[m] = __float2bfloat16_rn(lo);
        o_row[m + hv] = __float2bfloat16_rn(hi);
    }
}

// The chunks' maxima and denominators of a decode row put together into the row's own (`stats`), per head.
__global__ void __launch_bounds__(64)
talk_attention_stats_merge_kernel(const float* __restrict__ partial, int n_chunks, const int* __restrict__ tok_seq,
                                  const int* __restrict__ seq_slot, float* __restrict__ stats, int H, int dv, int sink,
                                  const float* __restrict__ sink_vals) {
    const int t = blockIdx.x;
    grid_dependents_launch();
    const int slot = seq_slot[tok_seq[t]];
    grid_dependency_wait();
    const float* base = partial + (size_t)t * n_chunks * H * (dv + 2);
    const size_t cs = (size_t)H * (dv + 2);
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float M = 0.f, Lsum = 0.f;
        if (slot >= 0) {
            const float* ph = base + (size_t)h * (dv + 2);
            const float z = sink_vals != nullptr ? sink_vals[h] : 0.f;
            M = sink ? z : -CUDART_INF_F;
            for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, ph[c * cs + dv]);
            Lsum = sink ? expf(z - M) : 0.f;
            for (int c = 0; c < n_chunks; ++c) {
                const float mc = ph[c * cs + dv];
                if (mc != -CUDART_INF_F) Lsum = fmaf(expf(mc - M), ph[c * cs + dv + 1], Lsum);
            }
        }
        stats[(size_t)t * 2 * H + 2 * h] = M;
        stats[(size_t)t * 2 * H + 2 * h + 1] = Lsum;
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_qkv_rotate_store(void* rows, int dtype, int row_elems, const int* tok_pos, const int* tok_seq,
                                        const int* seq_slot, const float* inv_qk, int rot, const float* inv_v, int T,
                                        int H, int G, int d, int dv, int with_kv, void* kpool, void* vpool,
                                        const int* page_table, int table_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1)) return fail("qkv_rotate_store: rotary width %d does not fit key size %d", rot, d);
    if (inv_v != nullptr && (dv & 1)) return fail("qkv_rotate_store: rotated values need an even size, found %d", dv);
    if (row_elems < H * d + (with_kv ? G * (d + dv) : 0)) return fail("qkv_rotate_store: rows of %d elements are too short", row_elems);
    if (with_kv && (!kpool || !vpool || !page_table || !seq_slot)) return fail("qkv_rotate_store: no cache line to store into");
    const dim3 grid(T), block(128);
    if (dtype == JANIS_F32)
        return launch_kernel("qkv_rotate_store", qkv_rotate_store_kernel<float>, grid, block, 0, stream, 1, (float*)rows,
                             row_elems, tok_pos, tok_seq, seq_slot, inv_qk, rot, inv_v, H, G, d, dv, with_kv, (float*)kpool,
                             (float*)vpool, page_table, table_stride);
    if (dtype == JANIS_BF16)
        return launch_kernel("qkv_rotate_store", qkv_rotate_store_kernel<bf16>, grid, block, 0, stream, 1, (bf16*)rows,
                             row_elems, tok_pos, tok_seq, seq_slot, inv_qk, rot, inv_v, H, G, d, dv, with_kv, (bf16*)kpool,
                             (bf16*)vpool, page_table, table_stride);
    return fail("qkv_rotate_store: unknown dtype %d", dtype);
}

static int talk_plain_tile(int H, int G, int d, int dv, size_t* bytes) {
    for (int kt = 32; kt >= 1; kt >>= 1) {
        const size_t b = talk_plain_smem_floats(H, G, d, dv, kt) * sizeof(float);
        if (b <= 200 * 1024) {
            *bytes = b;
            return kt;
        }
    }
    return 0;
}

static int talk_kernel_choice = 1;        // 1: the tensor-core kernel where it fits; 0: the plain kernel always

JANIS_EXPORT void janis_talk_attention_set_kernel(int which) { talk_kernel_choice = which; }

// The shape the tensor-core kernel runs a step with, or qr = 0 when it does not take the sizes.
static TalkMmaShape talk_mma_shape(int H, int G, int d, int dv, int one_row, size_t* bytes) {
    TalkMmaShape sh = {};
    if (H > 32 || d % 16 || dv % 8 || (dv & 1)) return sh;
    static const int order[6][2] = {{16, 64}, {16, 32}, {8, 64}, {8, 32}, {16, 16}, {8, 16}};
    for (int hg = 1; one_row && hg <= 8; hg *= 2) {
        // a decode step keeps one row of queries, scores and sums, so that several CTAs share an SM (tiles of
        // 64, 32 or 16 keys: the largest that leaves room for two CTAs, else the largest that fits)
        if (H % hg) break;
        for (int pass = 0; pass < 2; ++pass)
            for (int bn = 64; bn >= 16; bn >>= 1) {
                const TalkMmaLayout L = talk_mma_layout(H, G, d, dv, 1, bn, H / hg);
                if (L.total <= (size_t)(pass == 0 ? 110 : 220) * 1024) {
                    sh.qr = 1; sh.bn = bn; sh.rows = 1; sh.hg = hg;
                    *bytes = L.total;
                    return sh;
                }
            }
    }
    for (int hg = 1; hg <= 8; hg *= 2) {            // all heads' sums in one CTA where they fit, else the heads in groups
        if (H % hg) break;
        for (int i = 0; i < 6; ++i) {
            const int qr = order[i][0], bn = order[i][1];
            if (one_row && qr != 8) continue;
            const TalkMmaLayout L = talk_mma_layout(H, G, d, dv, qr, bn, H / hg);
            if (L.total <= 220 * 1024) {
                sh.qr = qr; sh.bn = bn; sh.rows = one_row ? 1 : qr; sh.hg = hg;
                *bytes = L.total;
                return sh;
            }
        }
    }
    return sh;
}

template <int HMAX>
static int talk_mma_launch(const void* q_rows, int q_row_elems, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                           const void* kpool, const void* vpool, const int* page_table, int table_stride,
                           const float* talk, const float* inv_v, void* out, float* partial, int n_chunks, int T,
                           TalkMmaShape sh, size_t bytes, cudaStream_t stream, const float* sink_vals, float* stats,
                           bool two_pass) {
    static size_t most = 0;
    if (bytes > most) {
        cudaError_t e = cudaFuncSetAttribute(talk_attention_mma_kernel<HMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return fail("talk_attention: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e));
        most = bytes;
    }
    const dim3 grid((T + sh.rows - 1) / sh.rows, (sh.chunk > 0 ? n_chunks : 1) * sh.hg), block(TALK_MMA_THREADS);
    // heads mixed after the softmax: a pass for the rows' maxima and denominators, then the pass of the weights
    for (int pass = two_pass ? 1 : 0; pass <= (two_pass ? 2 : 0); ++pass) {
        sh.mode = pass;
        if (launch_kernel("talk_attention", talk_attention_mma_kernel<HMAX>, grid, block, bytes, stream, 1, (const bf16*)q_rows,
                          q_row_elems, tok_pos, tok_seq, seq_slot, (const bf16*)kpool, (const bf16*)vpool, page_table,
                          table_stride, talk, inv_v, (bf16*)out, partial, sink_vals, stats, T, sh))
            return 1;
        if (sh.chunk == 0) continue;
        if (pass == 1) {
            if (launch_kernel("talk_attention_stats_merge", talk_attention_stats_merge_kernel, dim3(T), dim3(64), 0, stream, 1,
                              (const float*)partial, n_chunks, tok_seq, seq_slot, stats, sh.H, sh.dv, sh.sink, sink_vals))
                return 1;
        } else if (launch_kernel("talk_attention_merge", talk_attention_merge_kernel, dim3(T), dim3(128), 0, stream, 1,
                                 (const float*)partial, n_chunks, tok_pos, tok_seq, seq_slot, inv_v, (bf16*)out, sh.H, sh.dv,
                                 pass == 2 ? 0 : sh.sink, sink_vals)) {
            return 1;
        }
    }
    return 0;
}

JANIS_EXPORT int janis_talk_attention(const void* q_rows, int dtype, int q_row_elems, const int* tok_pos,
                                      const int* tok_seq, const int* seq_slot, const void* kpool, const void* vpool,
                                      const int* page_table, int table_stride, const float* talk, const float* inv_v,
                                      void* out, int T, int H, int G, int d, int dv, float scale, int block, int sink,
                                      int one_row, int max_keys, int n_chunks, float* partial, long long partial_floats,
                                      int window, float cap, const float* sink_vals, int mix_after, int v_in_keys,
                                      float* stats, long long stats_floats, int keep_first, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G) return fail("talk_attention: %d query heads do not divide over %d key/value heads", H, G);
    if (d <= 0 || dv <= 0) return fail("talk_attention: key size %d, value size %d", d, dv);
    if (inv_v != nullptr && (dv & 1)) return fail("talk_attention: rotated values need an even size, found %d", dv);
    if (q_row_elems < H * d) return fail("talk_attention: query rows of %d elements are too short", q_row_elems);
    if (block < 0) return fail("talk_attention: block size %d", block);
    if (window < 0) return fail("talk_attention: window %d", window);
    if (keep_first < 0 || (keep_first > 0 && (window <= 0 || block > 0)))
        return fail("talk_attention: %d kept first positions need a window and no blocks", keep_first);
    if (v_in_keys && (dv > d || inv_v != nullptr)) return fail("talk_attention: values of %d features do not lie in keys of %d", dv, d);
    if (sink_vals != nullptr && !sink) return fail("talk_attention: sink values without a sink");
    const bool two_pass = mix_after && talk != nullptr;       // (without a matrix there is nothing to mix: one pass)
    if (two_pass && (stats == nullptr || stats_floats < (long long)T * 2 * H))
        return fail("talk_attention: heads mixed after the softmax need %lld floats for the rows' maxima and denominators", (long long)T * 2 * H);
    if (v_in_keys) vpool = kpool;
    if (dtype == JANIS_BF16 && talk_kernel_choice == 1 && q_row_elems % 8 == 0 &&
        (((uintptr_t)q_rows | (uintptr_t)kpool | (uintptr_t)vpool) & 15) == 0) {
        size_t mma_bytes = 0;
        TalkMmaShape ms = talk_mma_shape(H, G, d, dv, one_row, &mma_bytes);
        if (ms.qr) {
            ms.H = H; ms.G = G; ms.d = d; ms.dv = dv; ms.block = block; ms.sink = sink ? 1 : 0; ms.scale = scale; ms.window = window; ms.keep_first = keep_first;
            ms.cap = cap; ms.mode = 0; ms.v_in_keys = v_in_keys ? 1 : 0;
            if (one_row && n_chunks > 1 && max_keys > 0 && partial != nullptr) {
                // a decode row's keys over n_chunks CTAs, each a whole number of tiles
                if (partial_floats < (long long)T * n_chunks * H * (dv + 2))
                    return fail("talk_attention: scratch of %lld floats is too small for %d rows in %d chunks", partial_floats, T, n_chunks);
                const int per = (max_keys + n_chunks - 1) / n_chunks;
                ms.chunk = (per + ms.bn - 1) / ms.bn * ms.bn;
            }
            if (H <= 8)
                return talk_mma_launch<8>(q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, table_stride,
                                          talk, inv_v, out, partial, n_chunks, T, ms, mma_bytes, stream, sink_vals, stats, two_pass);
            if (H <= 16)
                return talk_mma_launch<16>(q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, table_stride,
                                           talk, inv_v, out, partial, n_chunks, T, ms, mma_bytes, stream, sink_vals, stats, two_pass);
            return talk_mma_launch<32>(q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, kpool, vpool, page_table, table_stride,
                                       talk, inv_v, out, partial, n_chunks, T, ms, mma_bytes, stream, sink_vals, stats, two_pass);
        }
    }
    size_t bytes = 0;
    TalkShape sh;
    sh.H = H; sh.G = G; sh.d = d; sh.dv = dv; sh.block = block; sh.sink = sink ? 1 : 0; sh.scale = scale; sh.window = window; sh.keep_first = keep_first;
    sh.cap = cap; sh.mode = 0; sh.v_stride = v_in_keys ? d : dv;
    sh.kt = talk_plain_tile(H, G, d, dv, &bytes);
    if (sh.kt == 0) return fail("talk_attention: heads of these sizes do not fit shared memory (%d x %d, %d x %d)", H, d, G, dv);
    const dim3 grid(T), block_dim(256);
    if (dtype == JANIS_F32) {
        static size_t most_f = 0;
        if (bytes > most_f) {
            cudaError_t e = cudaFuncSetAttribute(talk_attention_plain_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return fail("talk_attention: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e));
            most_f = bytes;
        }
        for (int pass = two_pass ? 1 : 0; pass <= (two_pass ? 2 : 0); ++pass) {
            sh.mode = pass;
            if (launch_kernel("talk_attention", talk_attention_plain_kernel<float>, grid, block_dim, bytes, stream, 1,
                              (const float*)q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, (const float*)kpool,
                              (const float*)vpool, page_table, table_stride, talk, inv_v, (float*)out, sink_vals, stats, sh))
                return 1;
        }
        return 0;
    }
    if (dtype == JANIS_BF16) {
        static size_t most_b = 0;
        if (bytes > most_b) {
            cudaError_t e = cudaFuncSetAttribute(talk_attention_plain_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return fail("talk_attention: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e));
            most_b = bytes;
        }
        for (int pass = two_pass ? 1 : 0; pass <= (two_pass ? 2 : 0); ++pass) {
            sh.mode = pass;
            if (launch_kernel("talk_attention", talk_attention_plain_kernel<bf16>, grid, block_dim, bytes, stream, 1,
                              (const bf16*)q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, (const bf16*)kpool,
                              (const bf16*)vpool, page_table, table_stride, talk, inv_v, (bf16*)out, sink_vals, stats, sh))
                return 1;
        }
        return 0;
    }
    return fail("talk_attention: unknown dtype %d", dtype);
}
