// Attention of single rows over the paged cache, for decode steps: every row of the step is one query position of a
// sequence of its own, so the work is reading that sequence's keys and values once, and there is nothing for a matrix
// unit to share between rows.  The same mathematics as the kernels that take whole prompts (scores capped, a window, a
// sink in the denominator, the heads' weights mixed after the softmax, values that lie in the keys), in four launches:
//
//   scores   a CTA per (row, chunk of keys): s_h[j] = cap(scale q_h . k_kv(h)[j]) for every head, written out as floats,
//            and the chunk's maximum and sum of exponentials per head;
//   stats    per (row, head): the maximum M over the chunks (and the sink), 1 / L with L the sum of the chunks' sums
//            brought to M (and the sink's exponential); a warp's lanes take the chunks in turn;
//   values   a CTA per (row, chunk): w_h[j] = exp(s_h[j] - M_h) / L_h, mixed over the heads where a matrix is given,
//            p_h = sum_g M[h, g] w_g, and o_h = sum_j p_h[j] v_kv(h)[j] over the chunk's keys, as floats;
//   sum      per row: the chunks' o added in ascending order and rounded.
//
// Keys are read once and values once, 16 bytes a lane; the scores cross global memory as floats (a few megabytes).  A
// chunk's borders depend on the row's own first seen key and the chunk length, and every sum's order on the sizes, so a
// row's result does not depend on the rows beside it.  Scores, weights and sums are float whatever is stored.
#include "common.cuh"

#include <math_constants.h>

namespace janis {

constexpr int ROWS_THREADS = 256, ROWS_WARPS = ROWS_THREADS / 32;
constexpr int ROWS_HB = 8;          // query heads of one key/value head that a pass of the scores takes
constexpr int ROWS_VB = 4;          // and a pass of the values (2 where a key/value head serves no more)

struct RowsShape {
    int H, G, d, dv;
    int v_stride;       // elements between the values of neighbouring positions (dv, or d when the values lie in the keys)
    int window;         // keys are seen among the row's last `window` positions (0: all earlier ones)
    int keep_first;     // with a window: the sequence's first `keep_first` positions stay seen behind it
    int chunk;          // keys a CTA takes
    int n_chunks;       // CTAs a row
    int sink;           // 0 none; 1 a key of score 0 without a value; 2 learnt values
    int lanes;          // lanes of the scores' kernel that share a key's row
    float scale, cap;
};

constexpr int ROWS_FLIGHT = 8;      // 16-byte loads a thread has in flight (kept as they came: four registers each)

// 16 bytes as they came, and as floats
template <typename T> __device__ __forceinline__ void rows_unpack(const uint4& raw, float* out);
template <> __device__ __forceinline__ void rows_unpack<float>(const uint4& raw, float* out) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void rows_unpack<bf16>(const uint4& raw, float* out) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {       // a bfloat16 is the upper half of a float
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// The keys a row sees are counted through: the kept first positions that lie before the window, then first .. pos.
// A chunk takes the counts j0 .. j1; rows_key gives a count's position in the sequence.
struct RowsKeys { int first, kept; };
__device__ __forceinline__ RowsKeys rows_range(const RowsShape& sh, int pos, int c, int& j0, int& j1) {
    RowsKeys k;
    k.first = sh.window > 0 ? max(0, pos - sh.window + 1) : 0;
    k.kept = sh.window > 0 ? min(sh.keep_first, k.first) : 0;
    j0 = c * sh.chunk;
    j1 = min(k.kept + pos - k.first, j0 + sh.chunk - 1);
    return k;
}
__device__ __forceinline__ int rows_key(const RowsKeys& k, int n) { return n < k.kept ? n : k.first + n - k.kept; }

// scores [T, H, n_chunks * chunk], part [T, n_chunks, H, 2]
template <typename T>
__global__ void __launch_bounds__(ROWS_THREADS)
rows_scores_kernel(const T* __restrict__ q_rows, int q_row_elems, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, const T* __restrict__ kpool,
                   const int* __restrict__ page_table, int table_stride, RowsShape sh, float* __restrict__ scores,
                   float* __restrict__ part) {
    constexpr int V = Vec16<T>::N;
    extern __shared__ float rows_smem[];
    const int H = sh.H, G = sh.G, d = sh.d, rep = H / G;
    float* q_s = rows_smem;                         // the row's queries
    float* s_s = q_s + (size_t)H * (d + 8);         // the chunk's scores, head by head
    int* base_s = reinterpret_cast<int*>(s_s + (size_t)H * sh.chunk);      // where a key's row starts, in rows
    const int t = blockIdx.y, c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    int j0, j1;
    const RowsKeys keys = rows_range(sh, pos, c, j0, j1);
    grid_dependency_wait();
    float* prt = part + ((size_t)t * sh.n_chunks + c) * H * 2;
    if (slot < 0 || j0 > j1) {
        for (int h = tid; h < H; h += ROWS_THREADS) prt[2 * h] = -CUDART_INF_F, prt[2 * h + 1] = 0.f;
        return;
    }
    const int qs = d + 8;                           // (rows of the queries a little apart: heads fall on different banks)
    for (int i = tid; i < H * d; i += ROWS_THREADS) q_s[(size_t)(i / d) * qs + i % d] = to_float(q_rows[(size_t)t * q_row_elems + i]);
    const int n_keys = j1 - j0 + 1, n_pairs = n_keys * G;
    {
        const int* table = page_table + (size_t)slot * table_stride;
        for (int jj = tid; jj < n_keys; jj += ROWS_THREADS) {
            const int j = rows_key(keys, j0 + jj);
            base_s[jj] = table[j / JANIS_PAGE] * G * JANIS_PAGE + j % JANIS_PAGE;
        }
    }
    __syncthreads();
    // `lanes` neighbouring lanes share a (key, key/value head) pair and take its 16-byte pieces in turn, eight of them in
    // flight a lane; their partial sums meet in a butterfly.  Every lane of a warp runs every pass (the last pairs repeat).
    const int P = sh.lanes, sub = tid % P, n_slots = ROWS_THREADS / P, n_pieces = d / V;
    for (int pair0 = 0; pair0 < n_pairs; pair0 += n_slots) {
        const int mine = pair0 + tid / P, pair = mine < n_pairs ? mine : n_pairs - 1;
        const int jj = pair / G, g = pair % G;
        const T* krow = kpool + ((size_t)base_s[jj] + (size_t)g * JANIS_PAGE) * d;
        for (int hb = 0; hb < rep; hb += ROWS_HB) {
            float acc[ROWS_HB];
#pragma unroll
            for (int r = 0; r < ROWS_HB; ++r) acc[r] = 0.f;
            for (int i0 = sub; i0 < n_pieces; i0 += ROWS_FLIGHT * P) {
                uint4 raw[ROWS_FLIGHT];
#pragma unroll
                for (int u = 0; u < ROWS_FLIGHT; ++u) {
                    if (i0 + u * P < n_pieces) raw[u] = *reinterpret_cast<const uint4*>(krow + (size_t)(i0 + u * P) * V);
                }
#pragma unroll
                for (int u = 0; u < ROWS_FLIGHT; ++u) {
                    if (i0 + u * P < n_pieces) {
                        float x[V];
                        rows_unpack<T>(raw[u], x);
#pragma unroll
                        for (int r = 0; r < ROWS_HB; ++r) {
                            if (hb + r < rep) {
                                const float* qh = q_s + (size_t)(g * rep + hb + r) * qs + (size_t)(i0 + u * P) * V;
#pragma unroll
                                for (int e = 0; e < V; ++e) acc[r] = fmaf(qh[e], x[e], acc[r]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS_HB; ++r) {
                if (hb + r < rep) {
                    float v = acc[r];
                    for (int o = P >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    v *= sh.scale;
                    if (sh.cap > 0.f) v = sh.cap * tanhf(v / sh.cap);
                    if (sub == 0 && mine < n_pairs) s_s[(size_t)(g * rep + hb + r) * sh.chunk + jj] = v;
                }
            }
        }
    }
    __syncthreads();
    const size_t row_len = (size_t)sh.n_chunks * sh.chunk;
    for (int h = warp; h < H; h += ROWS_WARPS) {
        const float* s = s_s + (size_t)h * sh.chunk;
        float* dst = scores + ((size_t)t * H + h) * row_len + (size_t)c * sh.chunk;
        float m = -CUDART_INF_F;
        for (int jj = lane; jj < n_keys; jj += 32) {
            m = fmaxf(m, s[jj]);
            dst[jj] = s[jj];
        }
        m = warp_max(m);
        float l = 0.f;
        for (int jj = lane; jj < n_keys; jj += 32) l += expf(s[jj] - m);
        l = warp_sum(l);
        if (lane == 0) prt[2 * h] = m, prt[2 * h + 1] = l;
    }
}

// fin [T, H, 2]: the row's maximum and 1 / denominator per head; a warp per (row, head), a lane per chunk in turn, the
// lanes' sums met in a butterfly
__global__ void __launch_bounds__(128)
rows_stats_kernel(const float* __restrict__ part, const float* __restrict__ sink_values, RowsShape sh, int n_rows,
                  float* __restrict__ fin) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (u >= n_rows * sh.H) return;
    const int t = u / sh.H, h = u % sh.H;
    const float* p = part + (size_t)t * sh.n_chunks * sh.H * 2 + 2 * h;
    const float z = sh.sink == 2 ? sink_values[h] : 0.f;
    float M = sh.sink ? z : -CUDART_INF_F;
    for (int c = lane; c < sh.n_chunks; c += 32) M = fmaxf(M, p[(size_t)c * sh.H * 2]);
    M = warp_max(M);
    float L = 0.f;
    for (int c = lane; c < sh.n_chunks; c += 32) {
        const float m = p[(size_t)c * sh.H * 2], l = p[(size_t)c * sh.H * 2 + 1];
        if (l > 0.f) L += l * expf(m - M);
    }
    L = warp_sum(L);
    if (sh.sink) L += expf(z - M);
    if (lane == 0) {
        fin[2 * u] = M;
        fin[2 * u + 1] = L > 0.f ? 1.f / L : 0.f;
    }
}

// o_part [T, n_chunks, H, dv]
// VB: the query heads of one key/value head that a pass over the chunk's values takes
template <typename T, int VB>
__global__ void __launch_bounds__(ROWS_THREADS, VB <= 2 ? 3 : 2)
rows_values_kernel(const float* __restrict__ scores, const float* __restrict__ fin, const float* __restrict__ talk,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                   const T* __restrict__ vpool, const int* __restrict__ page_table, int table_stride, RowsShape sh,
                   float* __restrict__ o_part) {
    constexpr int V = Vec16<T>::N;
    extern __shared__ float rows_smem[];
    const int H = sh.H, G = sh.G, dv = sh.dv, rep = H / G, chunk = sh.chunk;
    float* w_s = rows_smem;                         // every head's own weights of the chunk's keys
    float* p_s = talk != nullptr ? w_s + (size_t)H * chunk : w_s;       // and the mixed ones
    float* red = p_s + (size_t)H * chunk;           // VB x V x ROWS_THREADS partial sums
    int* base_s = reinterpret_cast<int*>(red + (size_t)ROWS_THREADS * VB * V);    // where a key's row starts, in rows
    const int t = blockIdx.y, c = blockIdx.x, tid = threadIdx.x;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    int j0, j1;
    const RowsKeys keys = rows_range(sh, pos, c, j0, j1);
    grid_dependency_wait();
    if (slot < 0 || j0 > j1) return;                // (the sum leaves such chunks out)
    const int n_keys = j1 - j0 + 1;
    const int* table = page_table + (size_t)slot * table_stride;
    for (int jj = tid; jj < n_keys; jj += ROWS_THREADS) {
        const int j = rows_key(keys, j0 + jj);
        base_s[jj] = table[j / JANIS_PAGE] * G * JANIS_PAGE + j % JANIS_PAGE;
    }
    const size_t row_len = (size_t)sh.n_chunks * chunk;
    for (int i = tid; i < H * n_keys; i += ROWS_THREADS) {
        const int h = i / n_keys, jj = i % n_keys;
        const float s = scores[((size_t)t * H + h) * row_len + (size_t)c * chunk + jj];
        w_s[(size_t)h * chunk + jj] = expf(s - fin[((size_t)t * H + h) * 2]) * fin[((size_t)t * H + h) * 2 + 1];
    }
    __syncthreads();
    if (talk != nullptr) {
        for (int i = tid; i < H * n_keys; i += ROWS_THREADS) {
            const int h = i / n_keys, jj = i % n_keys;
            float s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(talk[h * H + g], w_s[(size_t)g * chunk + jj], s);
            p_s[(size_t)h * chunk + jj] = s;
        }
        __syncthreads();
    }
    // a unit is 16 bytes of one key/value head's features; the threads of a unit share the chunk's keys
    const int per_head = dv / V, n_units = G * per_head;
    const int share = n_units >= ROWS_THREADS ? 1 : ROWS_THREADS / n_units;
    float* out = o_part + ((size_t)t * sh.n_chunks + c) * H * dv;
    for (int u0 = 0; u0 < n_units; u0 += ROWS_THREADS / share) {
        const int u = u0 + tid % (ROWS_THREADS / share), sub = tid / (ROWS_THREADS / share);
        const bool live = u < n_units && sub < share;
        const int g = live ? u / per_head : 0, c0 = live ? (u % per_head) * V : 0;
        for (int hb = 0; hb < rep; hb += VB) {
            float acc[VB][V];
#pragma unroll
            for (int r = 0; r < VB; ++r)
#pragma unroll
                for (int e = 0; e < V; ++e) acc[r][e] = 0.f;
            if (live) {
                for (int jj = sub; jj < n_keys; jj += ROWS_FLIGHT * share) {      // keys in flight, added in ascending order
                    uint4 raw[ROWS_FLIGHT];
#pragma unroll
                    for (int k = 0; k < ROWS_FLIGHT; ++k) {
                        if (jj + k * share < n_keys)
                            raw[k] = *reinterpret_cast<const uint4*>(
                                vpool + ((size_t)base_s[jj + k * share] + (size_t)g * JANIS_PAGE) * sh.v_stride + c0);
                    }
#pragma unroll
                    for (int k = 0; k < ROWS_FLIGHT; ++k) {
                        if (jj + k * share < n_keys) {
                            float x[V];
                            rows_unpack<T>(raw[k], x);
#pragma unroll
                            for (int r = 0; r < VB; ++r) {
                                if (hb + r < rep) {
                                    const float p = p_s[(size_t)(g * rep + hb + r) * chunk + jj + k * share];
#pragma unroll
                                    for (int e = 0; e < V; ++e) acc[r][e] = fmaf(p, x[e], acc[r][e]);
                                }
                            }
                        }
                    }
                }
            }
            __syncthreads();                        // (red may still be read from the pass before)
#pragma unroll
            for (int r = 0; r < VB; ++r)
#pragma unroll
                for (int e = 0; e < V; ++e) red[(size_t)(r * V + e) * ROWS_THREADS + tid] = acc[r][e];
            __syncthreads();
            if (live && sub == 0) {
                for (int r = 0; r < VB; ++r) {
                    if (hb + r >= rep) break;
                    float sum[V];
#pragma unroll
                    for (int e = 0; e < V; ++e) sum[e] = 0.f;
                    for (int s2 = 0; s2 < share; ++s2) {
                        const int other = s2 * (ROWS_THREADS / share) + tid;
#pragma unroll
                        for (int e = 0; e < V; ++e) sum[e] += red[(size_t)(r * V + e) * ROWS_THREADS + other];
                    }
                    float* dst = out + (size_t)(g * rep + hb + r) * dv + c0;
#pragma unroll
                    for (int e = 0; e < V; e += 4) Vec16<float>::store(dst + e, sum + e);
                }
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(ROWS_THREADS)
rows_sum_kernel(const float* __restrict__ o_part, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                const int* __restrict__ seq_slot, RowsShape sh, T* __restrict__ out) {
    const int t = blockIdx.y, n = sh.H * sh.dv, i = (blockIdx.x * ROWS_THREADS + threadIdx.x) * 4;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    const int first = sh.window > 0 ? max(0, pos - sh.window + 1) : 0, kept = sh.window > 0 ? min(sh.keep_first, first) : 0;
    const int n_valid = slot < 0 ? 0 : min(sh.n_chunks, (kept + pos - first) / sh.chunk + 1);
    grid_dependency_wait();
    if (i >= n) return;
    const float* src = o_part + (size_t)t * sh.n_chunks * n + i;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < n_valid; c += 4) {
        float x[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (c + k < n_valid) Vec16<float>::load(src + (size_t)(c + k) * n, x[k]);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (c + k < n_valid) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[e] += x[k][e];
            }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) out[(size_t)t * n + i + e] = from_float<T>(s[e]);
}

struct RowsPlan {
    RowsShape sh;
    size_t scores, part, fin, o_part, total;        // offsets into the scratch, in floats
    size_t smem_scores, smem_values;
};

static RowsPlan rows_plan(int T, int H, int G, int d, int dv, int max_keys, int vec) {
    RowsPlan p = {};
    const int pages = (max_keys + 63) / 64;
    p.sh.chunk = 64 * ((pages + 63) / 64);
    p.sh.n_chunks = (max_keys + p.sh.chunk - 1) / p.sh.chunk;
    if (p.sh.n_chunks < 1) p.sh.n_chunks = 1;
    size_t at = 0;
    p.scores = at; at += (size_t)T * H * p.sh.n_chunks * p.sh.chunk;
    p.part = at;   at += (size_t)T * p.sh.n_chunks * H * 2;
    p.fin = at;    at += (size_t)T * H * 2;
    at = (at + 3) & ~(size_t)3;
    p.o_part = at; at += (size_t)T * p.sh.n_chunks * H * dv;
    p.total = at;
    p.smem_scores = ((size_t)H * (d + 8) + (size_t)H * p.sh.chunk + p.sh.chunk) * sizeof(float);
    // lanes that share a (key, key/value head) pair: a power of two, at least 2 (a whole 32-byte sector a load), so
    // that 64 keys fill the CTA, and no more than the row has pieces
    int lanes = 2;
    while (lanes < 32 && 64 * G * lanes * 2 <= ROWS_THREADS && lanes * 2 <= d / vec) lanes *= 2;
    if (d / vec < 2) lanes = 1;
    p.sh.lanes = lanes;
    p.smem_values = ((size_t)2 * H * p.sh.chunk + (size_t)ROWS_THREADS * ROWS_VB * vec + p.sh.chunk) * sizeof(float);
    return p;
}

}  // namespace janis

using namespace janis;

// Floats of scratch that `janis_talk_attention_rows` wants for such a step, or 0 when it does not take the sizes.
JANIS_EXPORT long long janis_talk_attention_rows_floats(int dtype, int T, int H, int G, int d, int dv, int max_keys) {
    const int vec = dtype == JANIS_F32 ? 4 : 8;
    if (T <= 0 || H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || max_keys <= 0) return 0;
    if (d % vec || dv % vec || H > 128) return 0;
    const RowsPlan p = rows_plan(T, H, G, d, dv, max_keys, vec);
    if (p.smem_scores > 160 * 1024 || p.smem_values > 160 * 1024) return 0;
    return (long long)p.total;
}

JANIS_EXPORT int janis_talk_attention_rows(const void* q_rows, int dtype, int q_row_elems, const int* tok_pos,
                                           const int* tok_seq, const int* seq_slot, const void* kpool, const void* vpool,
                                           const int* page_table, int table_stride, const float* talk, void* out, int T,
                                           int H, int G, int d, int dv, float scale, int sink, int max_keys, int window,
                                           float cap, const float* sink_values, int values_in_keys, float* scratch,
                                           long long scratch_floats, int keep_first, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && window <= 0)) return fail("talk_attention_rows: %d kept first positions need a window", keep_first);
    const long long want = janis_talk_attention_rows_floats(dtype, T, H, G, d, dv, max_keys);
    if (want <= 0) return fail("talk_attention_rows: sizes not taken (%d heads over %d, %d and %d features)", H, G, d, dv);
    if (scratch == nullptr || scratch_floats < want) return fail("talk_attention_rows: scratch of %lld floats, %lld wanted", scratch_floats, want);
    if (values_in_keys && dv > d) return fail("talk_attention_rows: values of %d features do not lie in keys of %d", dv, d);
    if (!values_in_keys && vpool == nullptr) return fail("talk_attention_rows: no values");
    if ((reinterpret_cast<uintptr_t>(kpool) | reinterpret_cast<uintptr_t>(vpool) | reinterpret_cast<uintptr_t>(scratch)) & 15)
        return fail("talk_attention_rows: pools and scratch start on 16-byte borders");
    const int vec = dtype == JANIS_F32 ? 4 : 8;
    RowsPlan p = rows_plan(T, H, G, d, dv, max_keys, vec);
    RowsShape& sh = p.sh;
    sh.H = H; sh.G = G; sh.d = d; sh.dv = dv;
    sh.v_stride = values_in_keys ? d : dv;
    sh.window = window;
    sh.keep_first = keep_first;
    sh.sink = sink ? (sink_values != nullptr ? 2 : 1) : 0;
    sh.scale = scale;
    sh.cap = cap;
    const dim3 grid(sh.n_chunks, T);
#define JANIS_ROWS(TT)                                                                                                 \
    {                                                                                                                  \
        static size_t most_s = 0, most_v = 0;                                                                          \
        if (p.smem_scores > most_s && p.smem_scores > 48 * 1024) {                                                     \
            if (cudaFuncSetAttribute(rows_scores_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem_scores) != cudaSuccess) \
                return fail("talk_attention_rows: shared memory of %zu bytes refused", p.smem_scores);                \
            most_s = p.smem_scores;                                                                                    \
        }                                                                                                              \
        auto values_kernel = H / G <= 2 ? rows_values_kernel<TT, 2> : rows_values_kernel<TT, ROWS_VB>;                 \
        if (p.smem_values > most_v && p.smem_values > 48 * 1024) {                                                     \
            if (cudaFuncSetAttribute(rows_values_kernel<TT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem_values) != cudaSuccess || \
                cudaFuncSetAttribute(rows_values_kernel<TT, ROWS_VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem_values) != cudaSuccess) \
                return fail("talk_attention_rows: shared memory of %zu bytes refused", p.smem_values);                \
            most_v = p.smem_values;                                                                                    \
        }                                                                                                              \
        const TT* vsrc = values_in_keys ? (const TT*)kpool : (const TT*)vpool;                                         \
        int rc = launch_kernel("talk_attention_rows (scores)", rows_scores_kernel<TT>, grid, dim3(ROWS_THREADS),       \
                               p.smem_scores, stream, 1, (const TT*)q_rows, q_row_elems, tok_pos, tok_seq, seq_slot,   \
                               (const TT*)kpool, page_table, table_stride, sh, scratch + p.scores, scratch + p.part);  \
        if (rc) return rc;                                                                                             \
        rc = launch_kernel("talk_attention_rows (stats)", rows_stats_kernel, dim3((T * H + 3) / 4), dim3(128), 0,      \
                           stream, 1, (const float*)(scratch + p.part), sink_values, sh, T, scratch + p.fin);          \
        if (rc) return rc;                                                                                             \
        rc = launch_kernel("talk_attention_rows (values)", values_kernel, grid,         dim3(ROWS_THREADS),           \
                           p.smem_values, stream, 1, (const float*)(scratch + p.scores),                               \
                           (const float*)(scratch + p.fin), talk, tok_pos, tok_seq, seq_slot, vsrc, page_table,        \
                           table_stride, sh, scratch + p.o_part);                                                      \
        if (rc) return rc;                                                                                             \
        return launch_kernel("talk_attention_rows (sum)", rows_sum_kernel<TT>, dim3((H * dv / 4 + ROWS_THREADS - 1) / ROWS_THREADS, T), dim3(ROWS_THREADS), 0, stream, \
                             1, (const float*)(scratch + p.o_part), tok_pos, tok_seq, seq_slot, sh, (TT*)out);         \
    }
    if (dtype == JANIS_F32) JANIS_ROWS(float)
    if (dtype == JANIS_BF16) JANIS_ROWS(bf16)
#undef JANIS_ROWS
    return fail("talk_attention_rows: unknown dtype %d", dtype);
}
