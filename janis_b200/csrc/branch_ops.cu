// Rows of the residual stream and of a layer's branches: the Dynamic Tanh norm, the RMS norm in groups that follows a
// scaled residual sum, the norm-and-accumulate of branches that run side by side, and a sigmoid gate on the heads of
// an attention.  All arithmetic is float.
#include "common.cuh"

#include <math_constants.h>

namespace janis {

// h[r] += res[r] (when res is given: the float residual sum, in place), then
// y[r] = tanh(alpha * h[src]) * w + b with src = rows[r] (or r): no statistics of the row are taken.
template <typename TR, typename TO>
__global__ void __launch_bounds__(256)
dyt_norm_kernel(float* __restrict__ h, const TR* __restrict__ res, const int* __restrict__ rows, float alpha,
                const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ y, int H) {
    const int r = blockIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    const int src = rows != nullptr ? rows[r] : r;
    float* hr = h + (size_t)src * H;
    TO* yr = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (res != nullptr) {
            v += to_float(res[(size_t)r * H + i]);
            hr[i] = v;
        }
        yr[i] = from_float<TO>(fmaf(tanhf(alpha * v), w[i], b[i]));
    }
}

// acc[r] = (first ? 0 : acc[r]) + share * x[r] / sqrt(mean(x[r]^2) + eps) * w
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_accumulate_kernel(const T* __restrict__ x, const float* __restrict__ w, float eps, float share,
                          float* __restrict__ acc, int first, int H) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    grid_dependents_launch();
    grid_dependency_wait();
    const T* xr = x + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_float(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = share / sqrtf(ss / (float)H + eps);
    float* ar = acc + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_float(xr[i]) * inv * w[i];
        ar[i] = first ? v : ar[i] + v;
    }
}

// RMS norm in groups: the row is cut into `groups` equal runs, each divided by sqrt(mean(run^2) + eps), and the whole
// multiplied by w.  With a residual: v = alpha h[r] + res[r], h[r] = norm(v) (the stream itself is normed, in place)
// and y[r] = h[r] rounded; without: y[r] = norm(h[src]) with src = rows[r] (or r), h untouched.
// A group's sum runs over the lanes of its warps and then over its warps in index order.
__device__ __forceinline__ void load4(const float* p, float* o) { Vec16<float>::load(p, o); }
__device__ __forceinline__ void load4(const bf16* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float* v) { Vec16<float>::store(p, v); }
__device__ __forceinline__ void store4(bf16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// VEC: four elements a load and a store (a group's length is a multiple of four, and so is every row's start)
template <typename TR, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
group_norm_kernel(float* __restrict__ h, const TR* __restrict__ res, const int* __restrict__ rows, float alpha,
                  const float* __restrict__ w, float eps, int groups, TO* __restrict__ y, int H) {
    extern __shared__ float gn_smem[];
    float* row_s = gn_smem;                 // the row
    float* inv_s = row_s + H;               // 1 / rms of each group
    float* scratch = inv_s + groups;        // a partial sum per warp
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    grid_dependents_launch();
    grid_dependency_wait();
    const int src = rows != nullptr ? rows[r] : r;
    float* hr = h + (size_t)src * H;
    if (VEC) {
        for (int i = tid * 4; i < H; i += blockDim.x * 4) {
            float v[4], a[4];
            load4(hr + i, v);
            if (res != nullptr) {
                load4(res + (size_t)r * H + i, a);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = fmaf(alpha, v[e], a[e]);
            }
            store4(row_s + i, v);
        }
    } else {
        for (int i = tid; i < H; i += blockDim.x) {
            float v = hr[i];
            if (res != nullptr) v = fmaf(alpha, v, to_float(res[(size_t)r * H + i]));
            row_s[i] = v;
        }
    }
    const int gs = H / groups;
    const int wpg = nwarp / groups > 0 ? nwarp / groups : 1;      // warps that share a group
    const int gpr = nwarp / wpg;                                  // groups summed side by side
    for (int g0 = 0; g0 < groups; g0 += gpr) {
        __syncthreads();
        const int g = g0 + warp / wpg, wi = warp % wpg;
        float ss = 0.f;
        if (g < groups && warp < gpr * wpg)
            for (int i = wi * 32 + lane; i < gs; i += wpg * 32) {
                const float v = row_s[g * gs + i];
                ss = fmaf(v, v, ss);
            }
        ss = warp_sum(ss);
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        if (tid < gpr && g0 + tid < groups) {
            float tot = 0.f;
            for (int k = 0; k < wpg; ++k) tot += scratch[tid * wpg + k];
            inv_s[g0 + tid] = 1.f / sqrtf(tot / (float)gs + eps);
        }
    }
    __syncthreads();
    if (VEC) {
        for (int i = tid * 4; i < H; i += blockDim.x * 4) {
            float v[4], ww[4];
            load4(row_s + i, v);
            load4(w + i, ww);
            const float inv = inv_s[i / gs];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = v[e] * inv * ww[e];
            if (res != nullptr) store4(hr + i, v);
            if (y != nullptr) store4(y + (size_t)r * H + i, v);
        }
    } else {
        for (int i = tid; i < H; i += blockDim.x) {
            const float v = row_s[i] * inv_s[i / gs] * w[i];
            if (res != nullptr) hr[i] = v;
            if (y != nullptr) y[(size_t)r * H + i] = from_float<TO>(v);
        }
    }
}

// y = h rounded to the activation type: what a sublayer reads when it reads the stream itself
__global__ void __launch_bounds__(256) round_rows_kernel(const float* __restrict__ h, bf16* __restrict__ y, size_t n) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __float2bfloat16_rn(h[i]);
}

// x[t, c] *= sigmoid(rows[t, g_off + c / per]): a gate per element (per = 1) or per run of `per` elements (a head)
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ rows, int row_elems, int g_off, int width, int per, size_t n) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width;
        const int c = (int)(i % width) / per;
        const float g = to_float(rows[t * row_elems + g_off + c]);
        x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-g)));
    }
}

// ---------------------------------------------------------------------------
// Mixture of experts: the router and the experts' activation.
//
// router, a warp per token over E logits z (float):  s = sigmoid(z), c = s + correction;  experts form n_groups equal
// groups of neighbours, a group's score is the sum of its two largest c, the best `keep` groups stay (ties: the
// lower index); among their experts the `top` of largest c are chosen (ties: the lower index); the chosen get
// w_e = s_e / (sum of the chosen s + 1e-20) * scale, every other expert 0.  With a shared gate, column E of z is
// its logit and column E of the output its sigmoid.  With `softmax` the scores are the softmax of z over all entries instead.  With
// n_identity > 0 the router scores that many entries more, behind the experts (no groups then); they have no column of
// their own in the output: the weights of the chosen ones add up in its last column.
// ---------------------------------------------------------------------------
constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& at) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > v || (ov == v && oa < at)) { v = ov; at = oa; }
    }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ z, const float* __restrict__ correction, int T, int E, int n_groups, int keep,
                 int top, float scale, int shared_gate, float* __restrict__ out, int n_identity, int softmax) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * ROUTE_WARPS + warp;
    const int N = E + n_identity;                    // entries the router scores: the experts, then the identity entries
    float* s = smem + (size_t)warp * (4 * N);        // scores
    float* c = s + N;                                // choice scores (minus infinity once out of the running)
    float* gs = c + N;                               // group scores
    float* mark = gs + N;                            // 1 for the chosen
    grid_dependents_launch();
    grid_dependency_wait();
    if (t >= T) return;
    const int cols_in = N + (shared_gate ? 1 : 0), cols_out = E + (shared_gate ? 1 : 0) + (n_identity ? 1 : 0), per = N / n_groups;
    const float* zr = z + (size_t)t * cols_in;
    float* o = out + (size_t)t * cols_out;
    float zmax = -CUDART_INF_F, zsum = 0.f;
    if (softmax) {
        for (int e = lane; e < N; e += 32) zmax = fmaxf(zmax, zr[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < N; e += 32) {
            const float v = expf(zr[e] - zmax);
            s[e] = v;
            zsum += v;
        }
        zsum = warp_sum(zsum);
    }
    for (int e = lane; e < N; e += 32) {
        const float v = softmax ? s[e] / zsum : 1.0f / (1.0f + expf(-zr[e]));
        s[e] = v;
        c[e] = v + correction[e];
        mark[e] = 0.f;
    }
    if (shared_gate && lane == 0) o[E] = 1.0f / (1.0f + expf(-zr[N]));
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -CUDART_INF_F, b = -CUDART_INF_F;      // the two largest
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = c[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the kept groups get +inf as a mark; the others' experts leave the running
        for (int k = 0; k < keep; ++k) {
            float v = -CUDART_INF_F;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float gv = gs[g];
                if (gv != CUDART_INF_F && (gv > v || (gv == v && g < at))) { v = gv; at = g; }
            }
            warp_argmax(v, at);
            __syncwarp();
            if (lane == 0 && at < n_groups) gs[at] = CUDART_INF_F;
            __syncwarp();
        }
        for (int e = lane; e < N; e += 32)
            if (gs[e / per] != CUDART_INF_F) c[e] = -CUDART_INF_F;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float v = -CUDART_INF_F;
        int at = 0x7fffffff;
        for (int e = lane; e < N; e += 32) {
            const float cv = c[e];
            if (cv > v || (cv == v && e < at)) { v = cv; at = e; }
        }
        warp_argmax(v, at);
        __syncwarp();
        if (at >= N) break;                          // nothing left in the running
        total += s[at];
        if (lane == 0) {
            c[at] = -CUDART_INF_F;
            mark[at] = 1.f;
        }
        __syncwarp();
    }
    const float f = scale / (total + 1e-20f);
    for (int e = lane; e < E; e += 32) o[e] = mark[e] != 0.f ? s[e] * f : 0.f;
    if (n_identity) {
        float id = 0.f;                              // the identity entries' weights add up: they all return the input
        for (int e = E + lane; e < N; e += 32)
            if (mark[e] != 0.f) id += s[e] * f;
        id = warp_sum(id);
        if (lane == 0) o[cols_out - 1] = id;
    }
}

// out[t, :] += w[t] y[t, :], w[t] = wts[t, w_col]: what the chosen identity entries of a mixture add to its output
template <typename T>
__global__ void __launch_bounds__(256)
moe_identity_add_kernel(T* __restrict__ out, const T* __restrict__ y, const float* __restrict__ wts, int wts_stride, int w_col,
                        int width, size_t n) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int V = Vec16<T>::N;
    if (width % V == 0 && (((uintptr_t)out | (uintptr_t)y) & 15) == 0) {
        // 16 bytes a thread; the pieces of a row share its weight
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V; i < n; i += (size_t)gridDim.x * blockDim.x * V) {
            const float w = wts[(i / width) * wts_stride + w_col];
            if (w == 0.f) continue;
            float a[V], b[V];
            Vec16<T>::load(out + i, a);
            Vec16<T>::load(y + i, b);
#pragma unroll
            for (int e = 0; e < V; ++e) a[e] = fmaf(w, b[e], a[e]);
            Vec16<T>::store(out + i, a);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float w = wts[(i / width) * wts_stride + w_col];
        if (w != 0.f) out[i] = from_float<T>(fmaf(w, to_float(y[i]), to_float(out[i])));
    }
}

// a[t, col] = w[t, e] * g sigmoid(alpha g) (u + up_add), g = min(gate, limit), u = clamp(up, -limit, limit), over the
// columns of all experts side by side (expert e: `ff` columns; then the shared expert's `shared_ff`); in gu an
// expert's gate columns are followed by its up columns.  Experts of weight 0 give exact zeros.
template <typename T>
__global__ void __launch_bounds__(256)
moe_expert_act_kernel(const T* __restrict__ gu, const float* __restrict__ wts, int E, int ff, float limit, int shared_ff,
                      float shared_limit, float alpha, T* __restrict__ out, size_t n, int wcols, float up_add) {
    const int total = E * ff + shared_ff;
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / total;
        const int col = (int)(i % total);
        int e, j, width;
        float lim;
        size_t base;
        if (col < E * ff) { e = col / ff; j = col % ff; width = ff; lim = limit; base = (size_t)2 * e * ff; }
        else { e = E; j = col - E * ff; width = shared_ff; lim = shared_limit; base = (size_t)2 * E * ff; }
        const float w = wts[t * wcols + e];
        float a = 0.f;
        if (w != 0.f) {
            const T* row = gu + t * (size_t)(2 * total) + base;
            const float g = fminf(to_float(row[j]), lim);
            const float u = fminf(fmaxf(to_float(row[width + j]), -lim), lim);
            a = w * (g / (1.0f + expf(-alpha * g))) * (u + up_add);
        }
        out[i] = from_float<T>(a);
    }
}

// The same, 16 bytes of columns a thread (the experts' widths are multiples of that many columns, so a thread's
// columns belong to one expert): gate and up are read 16 bytes at a time, the result is written so.
template <typename T>
__global__ void __launch_bounds__(256)
moe_expert_act_vec_kernel(const T* __restrict__ gu, const float* __restrict__ wts, int E, int ff, float limit, int shared_ff,
                          float shared_limit, float alpha, T* __restrict__ out, int T_rows, int wcols, float up_add) {
    constexpr int V = Vec16<T>::N;
    const int total = E * ff + shared_ff, per_row = total / V;
    grid_dependents_launch();
    grid_dependency_wait();
    for (int t = blockIdx.y; t < T_rows; t += gridDim.y) {
        const float* wrow = wts + (size_t)t * wcols;
        const T* grow = gu + (size_t)t * (2 * (size_t)total);
        T* orow = out + (size_t)t * total;
        for (int ch = blockIdx.x * blockDim.x + threadIdx.x; ch < per_row; ch += gridDim.x * blockDim.x) {
            const int col = ch * V;
            int e, j, width;
            float lim;
            size_t base;
            if (col < E * ff) { e = col / ff; j = col - e * ff; width = ff; lim = limit; base = (size_t)2 * e * ff; }
            else { e = E; j = col - E * ff; width = shared_ff; lim = shared_limit; base = (size_t)2 * E * ff; }
            const float w = wrow[e];
            float a[V];
#pragma unroll
            for (int i = 0; i < V; ++i) a[i] = 0.f;
            if (w != 0.f) {
                float gv[V], uv[V];
                Vec16<T>::load(grow + base + j, gv);
                Vec16<T>::load(grow + base + width + j, uv);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float g = fminf(gv[i], lim);
                    const float u = fminf(fmaxf(uv[i], -lim), lim);
                    a[i] = w * (g / (1.0f + expf(-alpha * g))) * (u + up_add);
                }
            }
            Vec16<T>::store(orow + col, a);
        }
    }
}

}  // namespace janis

using namespace janis;

static inline unsigned flat_grid(size_t n) {
    const size_t want = (n + 255) / 256;
    return (unsigned)(want < 148 * 16 ? (want ? want : 1) : 148 * 16);
}

JANIS_EXPORT int janis_dyt_norm(float* h, const void* res, int res_dtype, const int* rows, float alpha, const float* w,
                                const float* b, void* y, int y_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (res != nullptr && rows != nullptr) return fail("dyt_norm: a residual is added to all rows, not to chosen ones");
    const dim3 grid(R), block(H >= 1024 ? 256 : 128);
#define JANIS_DYT(TR, TO)                                                                                              \
    return launch_kernel("dyt_norm", dyt_norm_kernel<TR, TO>, grid, block, 0, stream, 1, h, (const TR*)res, rows, alpha, w, \
                         b, (TO*)y, H);
    const int rd = res != nullptr ? res_dtype : JANIS_F32;
    if (rd == JANIS_F32 && y_dtype == JANIS_F32) { JANIS_DYT(float, float) }
    if (rd == JANIS_F32 && y_dtype == JANIS_BF16) { JANIS_DYT(float, bf16) }
    if (rd == JANIS_BF16 && y_dtype == JANIS_F32) { JANIS_DYT(bf16, float) }
    if (rd == JANIS_BF16 && y_dtype == JANIS_BF16) { JANIS_DYT(bf16, bf16) }
#undef JANIS_DYT
    return fail("dyt_norm: unknown dtypes %d, %d", res_dtype, y_dtype);
}

JANIS_EXPORT int janis_rmsnorm_accumulate(const void* x, int dtype, const float* w, float eps, float share, float* acc,
                                          int first, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    const dim3 grid(R), block(H >= 1024 ? 256 : 128);
    if (dtype == JANIS_F32)
        return launch_kernel("rmsnorm_accumulate", rmsnorm_accumulate_kernel<float>, grid, block, 0, stream, 1,
                             (const float*)x, w, eps, share, acc, first, H);
    if (dtype == JANIS_BF16)
        return launch_kernel("rmsnorm_accumulate", rmsnorm_accumulate_kernel<bf16>, grid, block, 0, stream, 1,
                             (const bf16*)x, w, eps, share, acc, first, H);
    return fail("rmsnorm_accumulate: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_sigmoid_gate(void* x, const void* rows, int dtype, int row_elems, int g_off, int T, int width,
                                    int per, cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    if (per <= 0 || width % per) return fail("sigmoid_gate: runs of %d elements do not divide %d", per, width);
    if (g_off < 0 || g_off + width / per > row_elems) return fail("sigmoid_gate: %d gates at %d do not fit rows of %d", width / per, g_off, row_elems);
    const size_t n = (size_t)T * width;
    if (dtype == JANIS_F32)
        return launch_kernel("sigmoid_gate", sigmoid_gate_kernel<float>, dim3(flat_grid(n)), dim3(256), 0, stream, 1, (float*)x,
                             (const float*)rows, row_elems, g_off, width, per, n);
    if (dtype == JANIS_BF16)
        return launch_kernel("sigmoid_gate", sigmoid_gate_kernel<bf16>, dim3(flat_grid(n)), dim3(256), 0, stream, 1, (bf16*)x,
                             (const bf16*)rows, row_elems, g_off, width, per, n);
    return fail("sigmoid_gate: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_group_norm(float* h, const void* res, int res_dtype, const int* rows, float alpha, const float* w,
                                  float eps, int groups, void* y, int y_dtype, int R, int H, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (groups <= 0 || H % groups) return fail("group_norm: %d groups do not divide a row of %d", groups, H);
    if (res != nullptr && rows != nullptr) return fail("group_norm: a residual is added to all rows, not to chosen ones");
    if (res == nullptr && y == nullptr) return fail("group_norm: nothing to write");
    const size_t bytes = ((size_t)H + groups + 32) * sizeof(float);
    if (bytes > 200 * 1024) return fail("group_norm: a row of %d does not fit shared memory", H);
    const dim3 grid(R), block(H >= 1024 ? 256 : 128);
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = (H / groups) % 4 == 0 && aligned(h) && aligned(res) && aligned(w) && aligned(y);
#define JANIS_GN_V(TR, TO, VEC)                                                                                        \
    {                                                                                                                  \
        static size_t most = 0;                                                                                        \
        if (bytes > most && bytes > 48 * 1024) {                                                                       \
            cudaError_t e = cudaFuncSetAttribute(group_norm_kernel<TR, TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); \
            if (e != cudaSuccess) return fail("group_norm: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e)); \
            most = bytes;                                                                                              \
        }                                                                                                              \
        return launch_kernel("group_norm", group_norm_kernel<TR, TO, VEC>, grid, block, bytes, stream, 1, h, (const TR*)res, rows, \
                             alpha, w, eps, groups, (TO*)y, H);                                                        \
    }
#define JANIS_GN(TR, TO)                                                                                               \
    {                                                                                                                  \
        if (vec) JANIS_GN_V(TR, TO, true)                                                                              \
        JANIS_GN_V(TR, TO, false)                                                                                      \
    }
    const int rd = res != nullptr ? res_dtype : JANIS_F32, yd = y != nullptr ? y_dtype : JANIS_F32;
    if (rd == JANIS_F32 && yd == JANIS_F32) JANIS_GN(float, float)
    if (rd == JANIS_F32 && yd == JANIS_BF16) JANIS_GN(float, bf16)
    if (rd == JANIS_BF16 && yd == JANIS_F32) JANIS_GN(bf16, float)
    if (rd == JANIS_BF16 && yd == JANIS_BF16) JANIS_GN(bf16, bf16)
#undef JANIS_GN
#undef JANIS_GN_V
    return fail("group_norm: unknown dtypes %d, %d", res_dtype, y_dtype);
}

JANIS_EXPORT int janis_round_rows(const float* h, void* y, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    return launch_kernel("round_rows", round_rows_kernel, dim3(flat_grid(n)), dim3(256), 0, stream, 1, h, (bf16*)y, n);
}

JANIS_EXPORT int janis_moe_route(const float* z, const float* correction, int T, int E, int n_groups, int keep, int top,
                                 float scale, int shared_gate, float* out, int n_identity, int softmax, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int N = E + n_identity;
    if (E < 0 || n_identity < 0 || N <= 0 || N > 1024) return fail("moe_route: %d experts and %d identity entries (up to 1024 are taken)", E, n_identity);
    if (n_identity > 0 && n_groups != 1) return fail("moe_route: identity entries stand in no group");
    if (n_groups <= 0 || N % n_groups || keep <= 0 || keep > n_groups || top <= 0 || top > keep * (N / n_groups))
        return fail("moe_route: %d entries in %d groups, %d kept, %d chosen", N, n_groups, keep, top);
    const size_t bytes = (size_t)ROUTE_WARPS * 4 * N * sizeof(float);
    return launch_kernel("moe_route", moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32),
                         bytes, stream, 1, z, correction, T, E, n_groups, keep, top, scale, shared_gate, out, n_identity, softmax);
}

JANIS_EXPORT int janis_moe_identity_add(void* out, const void* y, int dtype, const float* wts, int wts_stride, int w_col, int T,
                                        int width, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (w_col < 0 || w_col >= wts_stride) return fail("moe_identity_add: column %d of %d", w_col, wts_stride);
    const size_t n = (size_t)T * width;
    if (dtype == JANIS_F32)
        return launch_kernel("moe_identity_add", moe_identity_add_kernel<float>, dim3(flat_grid(n)), dim3(256), 0, stream, 1,
                             (float*)out, (const float*)y, wts, wts_stride, w_col, width, n);
    if (dtype == JANIS_BF16)
        return launch_kernel("moe_identity_add", moe_identity_add_kernel<bf16>, dim3(flat_grid(n)), dim3(256), 0, stream, 1,
                             (bf16*)out, (const bf16*)y, wts, wts_stride, w_col, width, n);
    return fail("moe_identity_add: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_moe_expert_act(const void* gu, int dtype, const float* wts, int E, int ff, float limit, int shared_ff,
                                      float shared_limit, float alpha, void* out, int T, int wts_stride, float up_add,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    if (wts_stride <= 0) wts_stride = E + (shared_ff ? 1 : 0);
    const size_t n = (size_t)T * ((size_t)E * ff + shared_ff);
    const int v = dtype == JANIS_F32 ? 4 : 8;
    if (ff % v == 0 && shared_ff % v == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const int per_row = (E * ff + shared_ff) / v;
        const dim3 grid((per_row + 255) / 256, T < 65535 ? T : 65535), block(256);
        if (dtype == JANIS_F32)
            return launch_kernel("moe_expert_act", moe_expert_act_vec_kernel<float>, grid, block, 0, stream, 1, (const float*)gu,
                                 wts, E, ff, limit, shared_ff, shared_limit, alpha, (float*)out, T, wts_stride, up_add);
        if (dtype == JANIS_BF16)
            return launch_kernel("moe_expert_act", moe_expert_act_vec_kernel<bf16>, grid, block, 0, stream, 1, (const bf16*)gu,
                                 wts, E, ff, limit, shared_ff, shared_limit, alpha, (bf16*)out, T, wts_stride, up_add);
    }
    if (dtype == JANIS_F32)
        return launch_kernel("moe_expert_act", moe_expert_act_kernel<float>, dim3(flat_grid(n)), dim3(256), 0, stream, 1,
                             (const float*)gu, wts, E, ff, limit, shared_ff, shared_limit, alpha, (float*)out, n, wts_stride, up_add);
    if (dtype == JANIS_BF16)
        return launch_kernel("moe_expert_act", moe_expert_act_kernel<bf16>, dim3(flat_grid(n)), dim3(256), 0, stream, 1,
                             (const bf16*)gu, wts, E, ff, limit, shared_ff, shared_limit, alpha, (bf16*)out, n, wts_stride, up_add);
    return fail("moe_expert_act: unknown dtype %d", dtype);
}
