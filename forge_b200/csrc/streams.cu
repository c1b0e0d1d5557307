// A residual stream kept as S copies ("hyper-connections"): x [T, S, W] fp32.  Around a sublayer
//
//     u   = sum_s a[s] x_s                                   what the sublayer's norm reads
//     x_t <- sum_s m[s, t] x_s + b[t] y   (all t at once)    what the sublayer's output y does to the copies
//
// and the two meet in one pass: a sublayer's write is followed at once by the next sublayer's read and RMS norm, so the
// kernel that writes also leaves  norm(sum_t a'[t] x_t) * w  for the sublayer that follows.  Everything is fp32; every sum
// over the copies runs in the order s = 0, 1, ..., and the norm's sum over the row in the fixed tree of block_sum, so a
// token's numbers do not depend on what else the step brings.
//
//   streams_expand   x_s = e for every s (the embedding output enters all copies)
//   streams_mix      any of: the write (y given), the read + norm (a' and w given), on all rows or on chosen rows
#include "common.cuh"

namespace {

constexpr int kThreads = 256, kMaxStreams = 16;

__global__ void __launch_bounds__(kThreads)
streams_expand_kernel(const float* __restrict__ e, float* __restrict__ x, int S, int W) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const float* er = e + (size_t)blockIdx.x * W;
    float* xr = x + (size_t)blockIdx.x * S * W;
    for (int c = threadIdx.x; c < W; c += kThreads) {
        const float v = er[c];
        for (int s = 0; s < S; ++s) xr[(size_t)s * W + c] = v;
    }
}

// One CTA per row.  rows (or null) picks the tokens; with y the copies of the token are rewritten.  u (dynamic shared
// memory, W floats) holds what the norm reads between the two walks.  V = 4: rows of a multiple of four channels on 16-byte
// boundaries go four channels a load (every channel's arithmetic is what V = 1 does).
template <int V> struct Pack;
template <> struct Pack<1> { using type = float; };
template <> struct Pack<4> { using type = float4; };
__device__ __forceinline__ float& lane_of(float& v, int) { return v; }
__device__ __forceinline__ float& lane_of(float4& v, int i) { return (&v.x)[i]; }

template <typename TOut, int S, int V>
__global__ void __launch_bounds__(kThreads)
streams_mix_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ outc,
                   const float* __restrict__ in_next, const float* __restrict__ w_next, TOut* __restrict__ normed,
                   const int32_t* __restrict__ rows, int W, float eps) {
    using P = typename Pack<V>::type;
    extern __shared__ __align__(16) float u[];
    __shared__ float red[32];
    __shared__ float cm[S * S], cb[S], ca[S];
    forge::pdl_launch_dependents();
    if (threadIdx.x < S * S && mix) cm[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        cb[threadIdx.x] = outc ? outc[threadIdx.x] : 0.f;
        ca[threadIdx.x] = in_next ? in_next[threadIdx.x] : 0.f;
    }
    forge::pdl_wait();
    __syncthreads();
    const int t = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)t * S * W;
    const float* yr = y ? y + (size_t)t * W : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < W; c += kThreads * V) {
        P old[S], cur[S];
#pragma unroll
        for (int s = 0; s < S; ++s) old[s] = *reinterpret_cast<const P*>(xr + (size_t)s * W + c);
        if (yr) {
            P yv = *reinterpret_cast<const P*>(yr + c);
#pragma unroll
            for (int k = 0; k < S; ++k) {
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < S; ++s) a = fmaf(cm[s * S + k], lane_of(old[s], i), a);
                    lane_of(cur[k], i) = fmaf(cb[k], lane_of(yv, i), a);
                }
                *reinterpret_cast<P*>(xr + (size_t)k * W + c) = cur[k];
            }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) cur[s] = old[s];
        }
        if (in_next) {
#pragma unroll
            for (int i = 0; i < V; ++i) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) a = fmaf(ca[s], lane_of(cur[s], i), a);
                u[c + i] = a;
                ss = fmaf(a, a, ss);
            }
        }
    }
    if (!in_next) return;
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    TOut* o = normed + (size_t)blockIdx.x * W;
    for (int c = threadIdx.x; c < W; c += kThreads) o[c] = forge::from_float<TOut>(u[c] * inv * w_next[c]);
}

template <typename TOut, int S, int V>
cudaError_t launch_mix_v(cudaStream_t stream, int R, float* x, const float* y, const float* mix, const float* outc, const float* in_next,
                         const float* w_next, void* normed, const int32_t* rows, int W, float eps) {
    const size_t smem = in_next ? sizeof(float) * W : 0;
    if (smem > 48 * 1024) {
        static forge::PerDeviceFlag attr;
        bool& done = attr.current();
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(streams_mix_kernel<TOut, S, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            done = true;
        }
    }
    return forge::launch(streams_mix_kernel<TOut, S, V>, dim3(R), dim3(kThreads), smem, stream, 1, x, y, mix, outc, in_next, w_next,
                         (TOut*)normed, rows, W, eps);
}

template <typename TOut, int S>
cudaError_t launch_mix(cudaStream_t stream, int R, float* x, const float* y, const float* mix, const float* outc, const float* in_next,
                       const float* w_next, void* normed, const int32_t* rows, int W, float eps) {
    // four channels a load keep 8 S numbers in registers: up to four copies
    if constexpr (S <= 4) {
        if ((W & 3) == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0)
            return launch_mix_v<TOut, S, 4>(stream, R, x, y, mix, outc, in_next, w_next, normed, rows, W, eps);
    }
    return launch_mix_v<TOut, S, 1>(stream, R, x, y, mix, outc, in_next, w_next, normed, rows, W, eps);
}

}  // namespace

// e fp32 [T, W] -> x fp32 [T, S, W], every copy equal to e.
extern "C" int forge_streams_expand(const float* e, float* x, int T, int S, int W, cudaStream_t stream) {
    if (T < 0 || S <= 0 || W <= 0) return forge::fail(FORGE_ERR_ARG, "streams_expand: bad sizes T=%d S=%d W=%d", T, S, W);
    if (T == 0) return FORGE_OK;
    return forge::check_launch("streams_expand", forge::launch(streams_expand_kernel, dim3(T), dim3(kThreads), 0, stream, 1, e, x, S, W));
}

// x fp32 [T, S, W].  y fp32 [T, W] with mix fp32 [S, S] (indexed [from, to]) and outc fp32 [S], or all three null (nothing is
// written).  in_next fp32 [S] with w_next fp32 [W] and normed [R, W] of out_dtype, or all three null.  rows int32 [R] or
// null (R = T, every token in turn); rows go with y == null only.
extern "C" int forge_streams_mix(float* x, const float* y, const float* mix, const float* outc, const float* in_next,
                                 const float* w_next, void* normed, int out_dtype, const int32_t* rows, int R, int S, int W, float eps,
                                 cudaStream_t stream) {
    if (R < 0 || S <= 0 || W <= 0) return forge::fail(FORGE_ERR_ARG, "streams_mix: bad sizes R=%d S=%d W=%d", R, S, W);
    if (S > kMaxStreams) return forge::fail(FORGE_ERR_UNSUPPORTED, "streams_mix: %d copies of the stream (at most %d)", S, kMaxStreams);
    if ((y == nullptr) != (mix == nullptr) || (y == nullptr) != (outc == nullptr))
        return forge::fail(FORGE_ERR_ARG, "streams_mix: a write needs the sublayer's output, the mixing matrix and the output weights");
    if ((in_next == nullptr) != (w_next == nullptr) || (in_next == nullptr) != (normed == nullptr))
        return forge::fail(FORGE_ERR_ARG, "streams_mix: a read needs its weights, the norm's weights and an output");
    if (rows && y) return forge::fail(FORGE_ERR_ARG, "streams_mix: chosen rows are read, not written");
    if (sizeof(float) * (size_t)W > 200 * 1024) return forge::fail(FORGE_ERR_UNSUPPORTED, "streams_mix: rows of %d channels", W);
    if (R == 0 || (!y && !in_next)) return FORGE_OK;
    cudaError_t e = cudaSuccess;
#define FORGE_STREAMS_CASE(N) case N: FORGE_DISPATCH_DTYPE(out_dtype, TO, e = (launch_mix<TO, N>(stream, R, x, y, mix, outc, in_next, w_next, normed, rows, W, eps))); break;
    switch (S) {
        FORGE_STREAMS_CASE(1) FORGE_STREAMS_CASE(2) FORGE_STREAMS_CASE(3) FORGE_STREAMS_CASE(4) FORGE_STREAMS_CASE(5) FORGE_STREAMS_CASE(6)
        FORGE_STREAMS_CASE(7) FORGE_STREAMS_CASE(8) FORGE_STREAMS_CASE(9) FORGE_STREAMS_CASE(10) FORGE_STREAMS_CASE(11) FORGE_STREAMS_CASE(12)
        FORGE_STREAMS_CASE(13) FORGE_STREAMS_CASE(14) FORGE_STREAMS_CASE(15) FORGE_STREAMS_CASE(16)
    }
#undef FORGE_STREAMS_CASE
    return forge::check_launch("streams_mix", e);
}
