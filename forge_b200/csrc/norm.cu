// RMSNorm over rows of the fp32 residual stream:  y = x * rsqrt(mean(x^2) + eps) * w.
// Formula of the reference (src/operators/cuda/cuda_rms_norm.cu:10-36, src/operators/cpu/norm.cpp:98-112),
// but the sum of squares uses a fixed reduction tree instead of atomicAdd on one shared float, so a
// row's result never depends on timing or on the other rows of the batch.  All arithmetic is fp32;
// only the store rounds to the output type.  `rows` (optional) picks which input rows are normed:
// the final norm runs only on the rows whose logits are wanted.
#include "common.cuh"

namespace {

constexpr int kNormThreads = 128;

template <typename TOut> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
};

// One CTA per row.  With H a multiple of 4 a thread reads float4s (the first kKeep of them stay in registers
// for the second pass, beside the weights they meet there) and writes four outputs at a time; any other H goes
// element by element.
template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ out,
               const int32_t* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    constexpr int kKeep = 4;
    forge::pdl_launch_dependents();
    // the norm's weights do not depend on the kernel before: a thread's first kKeep float4s of them are read ahead of
    // the dependency wait instead of after the row's reduction, where the load's latency stood in the open
    float4 gain[kKeep];
    if ((H & 3) == 0) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            gain[i] = c < (H >> 2) ? reinterpret_cast<const float4*>(w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    forge::pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    TOut* o = out + (size_t)r * H;
    if ((H & 3) == 0) {
        const int n4 = H >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        float4 keep[kKeep];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            keep[i] = c < n4 ? x4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += (keep[i].x * keep[i].x + keep[i].y * keep[i].y) + (keep[i].z * keep[i].z + keep[i].w * keep[i].w);
        }
        for (int c = threadIdx.x + kKeep * kNormThreads; c < n4; c += kNormThreads) {
            const float4 v = x4[c];
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        ss = forge::block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = threadIdx.x + i * kNormThreads;
            if (c < n4) {
                const float4 g = gain[i];
                Pack4<TOut>::store(o + 4 * c, keep[i].x * inv * g.x, keep[i].y * inv * g.y, keep[i].z * inv * g.z, keep[i].w * inv * g.w);
            }
        }
        for (int c = threadIdx.x + kKeep * kNormThreads; c < n4; c += kNormThreads) {
            const float4 v = x4[c], g = w4[c];
            Pack4<TOut>::store(o + 4 * c, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
    }
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += kNormThreads) o[c] = forge::from_float<TOut>(xr[c] * inv * w[c]);
}

// Two norms of the same rows with the same eps and different weights (the two branches of a parallel block): one read
// of the residual stream, one reduction, two outputs.
template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_pair_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2, TOut* __restrict__ out1,
                    TOut* __restrict__ out2, int H, float eps) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const float* xr = x + (size_t)blockIdx.x * H;
    TOut* o1 = out1 + (size_t)blockIdx.x * H;
    TOut* o2 = out2 + (size_t)blockIdx.x * H;
    float ss = 0.f;
    if ((H & 3) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        for (int c = threadIdx.x; c < (H >> 2); c += kNormThreads) {
            const float4 v = x4[c];
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        ss = forge::block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (int c = threadIdx.x; c < (H >> 2); c += kNormThreads) {
            const float4 v = x4[c], g = reinterpret_cast<const float4*>(w1)[c], h = reinterpret_cast<const float4*>(w2)[c];
            Pack4<TOut>::store(o1 + 4 * c, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
            Pack4<TOut>::store(o2 + 4 * c, v.x * inv * h.x, v.y * inv * h.y, v.z * inv * h.z, v.w * inv * h.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < H; c += kNormThreads) ss = fmaf(xr[c], xr[c], ss);
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        o1[c] = forge::from_float<TOut>(xr[c] * inv * w1[c]);
        o2[c] = forge::from_float<TOut>(xr[c] * inv * w2[c]);
    }
}

// Layer norm with weight and bias:  y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b.  One CTA per row; the mean
// first, then the mean of the squared deviations from it (not E[x^2] - mean^2), both with the fixed reduction tree.
template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, TOut* __restrict__ out,
                 const int32_t* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    TOut* o = out + (size_t)r * H;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) s += xr[c];
    const float mean = forge::block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        const float d = xr[c] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(forge::block_sum(ss, red) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += kNormThreads) o[c] = forge::from_float<TOut>(fmaf((xr[c] - mean) * inv, w[c], b[c]));
}

// A sublayer's output y joins the stream through a norm of its own:  r <- r + mult * y / rms(y) * w_y, and, where the next
// sublayer's input norm follows at once, out = r / rms(r) * w_next of the new r in the same pass (w_next null: r only).
// One CTA per row; every sum runs over the row in the order of the fixed tree.
template <typename TOut>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ w_y, float* __restrict__ r, const float* __restrict__ w_next,
                   TOut* __restrict__ out, int H, float eps, float mult) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const float* yr = y + (size_t)blockIdx.x * H;
    float* rr = r + (size_t)blockIdx.x * H;
    TOut* o = out + (size_t)blockIdx.x * H;
    // rows of a multiple of four channels on 16-byte boundaries go four channels a load, eight loads in flight per thread (a step of
    // one token is one CTA: what it waits for is the memory's latency, once per load that depends on another)
    if ((H & 3) == 0 && (((uintptr_t)y | (uintptr_t)r | (uintptr_t)w_y | (uintptr_t)w_next) & 15) == 0) {
        const int H4 = H >> 2;
        const float4* y4 = reinterpret_cast<const float4*>(yr);
        float4* r4 = reinterpret_cast<float4*>(rr);
        const float4* wy4 = reinterpret_cast<const float4*>(w_y);
        const float4* wn4 = reinterpret_cast<const float4*>(w_next);
        float ss = 0.f;
#pragma unroll 8
        for (int c = threadIdx.x; c < H4; c += kNormThreads) {
            const float4 v = y4[c];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = forge::block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        float s2 = 0.f;
#pragma unroll 8
        for (int c = threadIdx.x; c < H4; c += kNormThreads) {
            const float4 a = y4[c], w = wy4[c];
            float4 v = r4[c];
            v.x = fmaf(mult, a.x * inv * w.x, v.x); v.y = fmaf(mult, a.y * inv * w.y, v.y);
            v.z = fmaf(mult, a.z * inv * w.z, v.z); v.w = fmaf(mult, a.w * inv * w.w, v.w);
            r4[c] = v;
            s2 = fmaf(v.x, v.x, s2); s2 = fmaf(v.y, v.y, s2); s2 = fmaf(v.z, v.z, s2); s2 = fmaf(v.w, v.w, s2);
        }
        if (w_next == nullptr) return;
        s2 = forge::block_sum(s2, red);
        const float inv2 = 1.0f / sqrtf(s2 / (float)H + eps);
#pragma unroll 8
        for (int c = threadIdx.x; c < H4; c += kNormThreads) {
            const float4 v = r4[c], w = wn4[c];
            o[4 * c] = forge::from_float<TOut>(v.x * inv2 * w.x);
            o[4 * c + 1] = forge::from_float<TOut>(v.y * inv2 * w.y);
            o[4 * c + 2] = forge::from_float<TOut>(v.z * inv2 * w.z);
            o[4 * c + 3] = forge::from_float<TOut>(v.w * inv2 * w.w);
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) ss = fmaf(yr[c], yr[c], ss);
    ss = forge::block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < H; c += kNormThreads) {
        const float v = fmaf(mult, yr[c] * inv * w_y[c], rr[c]);
        rr[c] = v;
        s2 = fmaf(v, v, s2);
    }
    if (w_next == nullptr) return;
    s2 = forge::block_sum(s2, red);
    const float inv2 = 1.0f / sqrtf(s2 / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += kNormThreads) o[c] = forge::from_float<TOut>(rr[c] * inv2 * w_next[c]);
}

}  // namespace

// y fp32 [R, H] (a sublayer's output), r fp32 [R, H] (the stream, updated in place), w_y fp32 [H]; w_next fp32 [H] and out
// [R, H] of out_dtype, or both null.
extern "C" int forge_rmsnorm_add(const float* y, const float* w_y, float* r, const float* w_next, void* out, int out_dtype, int R,
                                 int H, float eps, float mult, cudaStream_t stream) {
    if (R < 0 || H <= 0) return forge::fail(FORGE_ERR_ARG, "rmsnorm_add: bad sizes R=%d H=%d", R, H);
    if ((w_next == nullptr) != (out == nullptr)) return forge::fail(FORGE_ERR_ARG, "rmsnorm_add: the next norm needs its weight and its output");
    if (R == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(rmsnorm_add_kernel<TO>, dim3(R), dim3(kNormThreads), 0, stream, 1, y, w_y, r, w_next, (TO*)out, H, eps, mult));
    return forge::check_launch("rmsnorm_add", e);
}

extern "C" int forge_layernorm(const float* x, const float* w, const float* b, void* out, int out_dtype, const int32_t* rows, int R,
                               int H, float eps, cudaStream_t stream) {
    if (R < 0 || H <= 0) return forge::fail(FORGE_ERR_ARG, "layernorm: bad sizes R=%d H=%d", R, H);
    if (R == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(layernorm_kernel<TO>, dim3(R), dim3(kNormThreads), 0, stream, 1, x, w, b, (TO*)out, rows, H, eps));
    return forge::check_launch("layernorm", e);
}

extern "C" int forge_rmsnorm_pair(const float* x, const float* w1, const float* w2, void* out1, void* out2, int out_dtype, int R, int H,
                                  float eps, cudaStream_t stream) {
    if (R < 0 || H <= 0) return forge::fail(FORGE_ERR_ARG, "rmsnorm_pair: bad sizes R=%d H=%d", R, H);
    if (R == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(rmsnorm_pair_kernel<TO>, dim3(R), dim3(kNormThreads), 0, stream, 1, x, w1, w2, (TO*)out1, (TO*)out2, H, eps));
    return forge::check_launch("rmsnorm_pair", e);
}

extern "C" int forge_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int32_t* rows,
                             int R, int H, float eps, cudaStream_t stream) {
    if (R < 0 || H <= 0) return forge::fail(FORGE_ERR_ARG, "rmsnorm: bad sizes R=%d H=%d", R, H);
    if (R == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(out_dtype, TO,
        e = forge::launch(rmsnorm_kernel<TO>, dim3(R), dim3(kNormThreads), 0, stream, 1, x, w, (TO*)out, rows, H, eps));
    return forge::check_launch("rmsnorm", e);
}
