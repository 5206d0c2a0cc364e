// Several copies of the residual stream that the sublayers read and write through small learnt maps
// (hyper-connections).  The stream is float [rows, S, W], a token's S copies side by side.  For a sublayer with the
// vectors a, b [S] and the matrix M [S, S] (indexed [from, to]):
//
//   read:    u[t]     = sum_s a[s] x[t, s]                       y = u / sqrt(mean(u^2) + eps) * w   (w holds offset + weight)
//   write:   x[t, k] <- sum_s M[s, k] x[t, s] + b[k] r[t]        all k from the old copies; r is the sublayer's output
//
// `hc_update` does the write and, when the next sublayer's a and w are given, that sublayer's read in the same pass
// over the row.  `hc_spread` makes the S copies of the embedding's rows.  All sums are float, in an order fixed by
// the sizes alone; a CTA owns a row.
#include "common.cuh"

namespace janis {

constexpr int HC_MAX = 8;          // copies of the stream

__global__ void __launch_bounds__(256)
hc_spread_kernel(const float* __restrict__ x, float* __restrict__ h, int S, int W, size_t n) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / W;
        const int c = (int)(i % W);
        const float v = x[i];
        for (int s = 0; s < S; ++s) h[(t * S + s) * W + c] = v;
    }
}

// four neighbouring elements at once: 16 bytes of floats, 8 of bfloat16
__device__ __forceinline__ void load4(const float* p, float (&y)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    y[0] = v.x; y[1] = v.y; y[2] = v.z; y[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&y)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    y[0] = __uint_as_float(v.x << 16); y[1] = __uint_as_float(v.x & 0xffff0000u);
    y[2] = __uint_as_float(v.y << 16); y[3] = __uint_as_float(v.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&y)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(y[0], y[1], y[2], y[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&y)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T>
__global__ void __launch_bounds__(256)
hc_read_norm_kernel(const float* __restrict__ h, const int* __restrict__ rows, const float* __restrict__ a,
                    const float* __restrict__ w, float eps, T* __restrict__ out, int S, int W) {
    extern __shared__ __align__(16) float hc_u[];
    __shared__ float scratch[32];
    const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    grid_dependents_launch();
    float av[HC_MAX];
#pragma unroll
    for (int s = 0; s < HC_MAX; ++s) av[s] = (a != nullptr && s < S) ? a[s] : 1.f;
    grid_dependency_wait();
    const size_t row = rows != nullptr ? (size_t)rows[r] : (size_t)r;
    const float* x = h + row * S * W;
    float ss = 0.f;
    T* o = out + (size_t)r * W;
    const bool vec = (W & 3) == 0 && (((uintptr_t)h | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
    if (vec) {
        // (the sums run in the same order per element as below: a row's result does not depend on the path)
        for (int c = tid * 4; c < W; c += nt * 4) {
            float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < HC_MAX; ++s)
                if (s < S) {
                    float v[4];
                    load4(x + (size_t)s * W + c, v);
#pragma unroll
                    for (int e = 0; e < 4; ++e) u[e] = fmaf(av[s], v[e], u[e]);
                }
            store4(hc_u + c, u);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(u[e], u[e], ss);
        }
    } else {
        for (int c = tid; c < W; c += nt) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX; ++s)
                if (s < S) u = fmaf(av[s], x[(size_t)s * W + c], u);
            hc_u[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)W + eps);
    if (vec) {
        for (int c = tid * 4; c < W; c += nt * 4) {
            float u[4], wv[4];
            load4(hc_u + c, u);
            load4(w + c, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) u[e] = u[e] * inv * wv[e];
            store4(o + c, u);
        }
        return;
    }
    for (int c = tid; c < W; c += nt) o[c] = from_float<T>(hc_u[c] * inv * w[c]);
}

// (SMAX: a compile-time bound on the copies, 2, 4 or 8: the loops over the copies are unrolled to it, and what a thread
// keeps in registers follows)
template <typename T, typename TO, int SMAX>
__global__ void __launch_bounds__(256)
hc_update_kernel(float* __restrict__ h, const T* __restrict__ res, const float* __restrict__ M, const float* __restrict__ b,
                 const float* __restrict__ a_next, const float* __restrict__ w_next, float eps_next,
                 TO* __restrict__ out, int S, int W) {
    extern __shared__ __align__(16) float hc_u[];
    __shared__ float scratch[32];
    __shared__ float m_s[HC_MAX * HC_MAX], b_s[HC_MAX], a_s[HC_MAX];
    const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    grid_dependents_launch();
    if (tid < S * S) m_s[tid] = M[tid];
    if (tid < S) {
        b_s[tid] = b[tid];
        a_s[tid] = a_next != nullptr ? a_next[tid] : 0.f;
    }
    __syncthreads();
    grid_dependency_wait();
    float* x = h + (size_t)r * S * W;
    const T* rr = res + (size_t)r * W;
    const bool read = w_next != nullptr;
    float ss = 0.f;
    const bool vec = (W & 3) == 0 && (((uintptr_t)h | (uintptr_t)res | (uintptr_t)out | (uintptr_t)w_next) & 15) == 0;
    for (int c = tid * 4; vec && c < W; c += nt * 4) {
        // four elements a thread: every copy 16 bytes a load and a store; the sums per element in the order of the loop below
        float y[4], fresh[SMAX][4];
        load4(rr + c, y);
#pragma unroll
        for (int k = 0; k < SMAX; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) fresh[k][e] = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) {
                float old[4];
                load4(x + (size_t)s * W + c, old);
#pragma unroll
                for (int k = 0; k < SMAX; ++k)
                    if (k < S) {
                        const float m = m_s[s * S + k];
#pragma unroll
                        for (int e = 0; e < 4; ++e) fresh[k][e] = fmaf(m, old[e], fresh[k][e]);
                    }
            }
        float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < SMAX; ++k)
            if (k < S) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    fresh[k][e] = fmaf(b_s[k], y[e], fresh[k][e]);
                    u[e] = fmaf(a_s[k], fresh[k][e], u[e]);
                }
                store4(x + (size_t)k * W + c, fresh[k]);
            }
        if (read) {
            store4(hc_u + c, u);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(u[e], u[e], ss);
        }
    }
    for (int c = tid; !vec && c < W; c += nt) {
        float old[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) old[s] = s < S ? x[(size_t)s * W + c] : 0.f;
        const float y = to_float(rr[c]);
        float u = 0.f;
#pragma unroll
        for (int k = 0; k < SMAX; ++k)
            if (k < S) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(m_s[s * S + k], old[s], v);
                v = fmaf(b_s[k], y, v);
                x[(size_t)k * W + c] = v;
                u = fmaf(a_s[k], v, u);
            }
        if (read) {
            hc_u[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!read) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)W + eps_next);
    TO* o = out + (size_t)r * W;
    if (vec) {
        for (int c = tid * 4; c < W; c += nt * 4) {
            float u[4], wv[4];
            load4(hc_u + c, u);
            load4(w_next + c, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) u[e] = u[e] * inv * wv[e];
            store4(o + c, u);
        }
        return;
    }
    for (int c = tid; c < W; c += nt) o[c] = from_float<TO>(hc_u[c] * inv * w_next[c]);
}

}  // namespace janis

using namespace janis;

static int hc_check(const char* what, int S, int W, size_t* bytes) {
    if (S < 1 || S > HC_MAX) return fail("%s: %d copies of the stream (1 to %d are taken)", what, S, HC_MAX);
    if (W < 1) return fail("%s: width %d", what, W);
    *bytes = (size_t)W * sizeof(float);
    if (*bytes > 48 * 1024) return fail("%s: rows of %d floats do not fit shared memory", what, W);
    return 0;
}

JANIS_EXPORT int janis_hc_spread(const float* x, float* h, int T, int S, int W, cudaStream_t stream) {
    if (T <= 0) return 0;
    size_t bytes;
    if (hc_check("hc_spread", S, W, &bytes)) return 1;
    const size_t n = (size_t)T * W, want = (n + 255) / 256;
    return launch_kernel("hc_spread", hc_spread_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, stream, 1,
                         x, h, S, W, n);
}

JANIS_EXPORT int janis_hc_read_norm(const float* h, const int* rows, const float* a, const float* w, float eps, void* out,
                                    int out_dtype, int R, int S, int W, cudaStream_t stream) {
    if (R <= 0) return 0;
    size_t bytes;
    if (hc_check("hc_read_norm", S, W, &bytes)) return 1;
    const dim3 grid(R), block(W >= 1024 ? 256 : 128);
    if (out_dtype == JANIS_F32)
        return launch_kernel("hc_read_norm", hc_read_norm_kernel<float>, grid, block, bytes, stream, 1, h, rows, a, w, eps,
                             (float*)out, S, W);
    if (out_dtype == JANIS_BF16)
        return launch_kernel("hc_read_norm", hc_read_norm_kernel<bf16>, grid, block, bytes, stream, 1, h, rows, a, w, eps,
                             (bf16*)out, S, W);
    return fail("hc_read_norm: unknown dtype %d", out_dtype);
}

JANIS_EXPORT int janis_hc_update(float* h, const void* res, int dtype, const float* M, const float* b, const float* a_next,
                                 const float* w_next, float eps_next, void* out, int R, int S, int W, cudaStream_t stream) {
    if (R <= 0) return 0;
    size_t bytes;
    if (hc_check("hc_update", S, W, &bytes)) return 1;
    if ((a_next == nullptr) != (w_next == nullptr) || (w_next != nullptr && out == nullptr))
        return fail("hc_update: the next sublayer's read needs its vector, its norm's weight and a place for the result");
    const dim3 grid(R), block(W >= 1024 ? 256 : 128);
#define JANIS_HC_UPDATE(TT, SMAX)                                                                                      \
    return launch_kernel("hc_update", hc_update_kernel<TT, TT, SMAX>, grid, block, bytes, stream, 1, h, (const TT*)res, M, b, \
                         a_next, w_next, eps_next, (TT*)out, S, W);
    if (dtype == JANIS_F32) {
        if (S <= 2) JANIS_HC_UPDATE(float, 2)
        if (S <= 4) JANIS_HC_UPDATE(float, 4)
        JANIS_HC_UPDATE(float, 8)
    }
    if (dtype == JANIS_BF16) {
        if (S <= 2) JANIS_HC_UPDATE(bf16, 2)
        if (S <= 4) JANIS_HC_UPDATE(bf16, 4)
        JANIS_HC_UPDATE(bf16, 8)
    }
#undef JANIS_HC_UPDATE
    return fail("hc_update: unknown dtype %d", dtype);
}
