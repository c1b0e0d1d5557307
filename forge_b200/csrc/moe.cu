// A feed-forward made of many small gated feed-forwards ("experts") of which a router picks a few per token.
//
//   route       z = Wr x in fp32, score = sigmoid(z) (or softmax over the experts), the `top` largest scores (the lower index
//               wins a tie) are the token's experts and, as they are or divided by their sum, its weights.  Options: experts are
//               ranked by score + correction_e (the weights stay the scores); the experts are cut into `groups` consecutive blocks
//               of equal size, a block is ranked by the largest ranking number in it, and only the `keep` best blocks' experts
//               take part; the weights are multiplied by a factor
//   by pairs    every (token, chosen expert) pair on its own: act = act_fn(Wg_e x) * (Wu_e x), then for every token
//               y = sum over its experts, in the order the router chose them, of weight * Wd_e act.  Everything is read from
//               device memory, so the path can be replayed in a CUDA graph; it is the path of steps with few tokens
//   sorted      for steps of many tokens: the pairs are ranked by (expert, token) so that each expert's tokens are
//               consecutive rows, the rows go through ordinary matrix products expert by expert, and a last kernel adds a
//               token's experts up in the router's order.  The rows lie packed (the caller reads the counts) or, for steps
//               that must not wait for the device, with room for a step's tokens per expert: expert e's rows from e * cap
//               on, the products of an expert without rows skipped on the device by its count
//
// Router arithmetic is fp32 whatever the activations' type.  Every sum has a fixed order: a dot product is dealt to the
// lanes of a warp by index and summed by the butterfly, a token's experts are added in the order of their scores.
#include <algorithm>
#include <type_traits>
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf(float x) { return x * sigmoidf(x); }

// A CTA of 8 warps per token: the warps take the experts in turn (a lane sums its channels in order, 8 neighbours at a time
// where the rows allow 16-byte loads, then the butterfly), thread 0 ranks the scores in shared memory [E].
template <typename TA>
__device__ __forceinline__ float route_dot(const TA* __restrict__ xr, const float* __restrict__ w, int W, int lane) {
    float a = 0.f;
    for (int c = lane; c < W; c += 32) a = fmaf(forge::to_float(xr[c]), w[c], a);
    return a;
}
template <>
__device__ __forceinline__ float route_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ xr, const float* __restrict__ w, int W, int lane) {
    float a = 0.f;
    if ((W & 7) == 0 && (((uintptr_t)xr) & 15) == 0 && (((uintptr_t)w) & 15) == 0) {
#pragma unroll 4
        for (int c = lane * 8; c < W; c += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
            const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 x0 = __bfloat1622float2(p[0]), x1 = __bfloat1622float2(p[1]), x2 = __bfloat1622float2(p[2]), x3 = __bfloat1622float2(p[3]);
            a = fmaf(x0.x, w0.x, a); a = fmaf(x0.y, w0.y, a); a = fmaf(x1.x, w0.z, a); a = fmaf(x1.y, w0.w, a);
            a = fmaf(x2.x, w1.x, a); a = fmaf(x2.y, w1.y, a); a = fmaf(x3.x, w1.z, a); a = fmaf(x3.y, w1.w, a);
        }
        return a;
    }
    for (int c = lane; c < W; c += 32) a = fmaf(__bfloat162float(xr[c]), w[c], a);
    return a;
}

constexpr int kRouteThreads = 256;

template <typename TA>
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const TA* __restrict__ x, const float* __restrict__ Wr, int32_t* __restrict__ idx, float* __restrict__ wts, int T,
                 int W, int E, int top, int softmax, int renorm, const float* __restrict__ corr, int groups, int keep, float factor) {
    extern __shared__ float sc[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x;
    float* s = sc;
    const TA* xr = x + (size_t)t * W;
    for (int e = warp; e < E; e += kRouteThreads / 32) {
        const float a = forge::warp_sum(route_dot(xr, Wr + (size_t)e * W, W, lane));
        if (lane == 0) s[e] = a;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (softmax) {
            float m = -INFINITY, sum = 0.f;
            for (int e = 0; e < E; ++e) m = fmaxf(m, s[e]);
            for (int e = 0; e < E; ++e) { s[e] = expf(s[e] - m); sum += s[e]; }
            for (int e = 0; e < E; ++e) s[e] /= sum;
        } else {
            for (int e = 0; e < E; ++e) s[e] = sigmoidf(s[e]);
        }
        // ch: what the choice is made by (the scores themselves unless a correction or groups say otherwise)
        float* ch = s;
        if (corr != nullptr || groups > 1) {
            ch = s + E;
            for (int e = 0; e < E; ++e) ch[e] = corr ? s[e] + corr[e] : s[e];
        }
        if (groups > 1) {
            float* gs = ch + E;                      // a block's rank: the largest ranking number in it
            const int per = E / groups;
            for (int g = 0; g < groups; ++g) {
                float b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, ch[e]);
                gs[g] = b;
            }
            // the `keep` best groups stay (the lower index wins a tie); a kept group is marked by NaN, which no comparison picks again
            for (int k = 0; k < keep; ++k) {
                int best = -1;
                float bv = -INFINITY;
                for (int g = 0; g < groups; ++g)
                    if (gs[g] == gs[g] && (best < 0 || gs[g] > bv)) { bv = gs[g]; best = g; }
                if (best >= 0) gs[best] = __int_as_float(0x7fc00000);
            }
            for (int g = 0; g < groups; ++g)
                if (gs[g] == gs[g])
                    for (int e = g * per; e < (g + 1) * per; ++e) ch[e] = -INFINITY;
        }
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (ch[e] > bv) { bv = ch[e]; best = e; }
            idx[(size_t)t * top + k] = best;
            wts[(size_t)t * top + k] = s[best];
            total += s[best];
            ch[best] = -INFINITY;
        }
        for (int k = 0; k < top; ++k) {
            float w = wts[(size_t)t * top + k];
            if (renorm) w /= total;
            wts[(size_t)t * top + k] = w * factor;
        }
    }
}

// dot of a weight row (global) with a vector in shared memory, dealt to the lanes by index; the same order whatever the type
template <typename TW>
__device__ __forceinline__ float lane_dot(const TW* __restrict__ w, const float* __restrict__ xs, int n, int lane) {
    float a = 0.f;
    for (int c = lane; c < n; c += 32) a = fmaf(forge::to_float(w[c]), xs[c], a);
    return a;
}
template <>
__device__ __forceinline__ float lane_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ xs, int n, int lane) {
    float a = 0.f;
    if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int c = lane * 8; c < n; c += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + c);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                a = fmaf(f.x, xs[c + 2 * i], a);
                a = fmaf(f.y, xs[c + 2 * i + 1], a);
            }
        }
        return a;
    }
    for (int c = lane; c < n; c += 32) a = fmaf(__bfloat162float(w[c]), xs[c], a);
    return a;
}

constexpr int kPairOutputs = 32;          // outputs per CTA of the expert-by-expert kernel (8 per warp)
constexpr int kPairTile = 16;             // outputs per CTA of the kernels that take every pair on its own (4 per warp, all at once)

// R dot products at once, each summed exactly as lane_dot sums it, so that a lane has R 16-byte loads in flight instead of one:
// rows w[r] against the vectors xs[r / XG] in shared memory (XG consecutive rows share a vector).
template <typename TW, int R, int XG, int DEEP = 1>
__device__ __forceinline__ void lane_dot_rows(const TW* const (&w)[R], const float* const (&xs)[R / XG], int n, int lane, float (&a)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) a[r] = 0.f;
    bool vec = std::is_same<TW, __nv_bfloat16>::value && (n & 7) == 0;
#pragma unroll
    for (int r = 0; r < R; ++r) vec = vec && (((uintptr_t)w[r]) & 15) == 0;
    if (vec) {
        // DEEP pieces of every row are asked for before the first is used (where few CTAs fit an SM, more bytes have to be in
        // flight per lane); a row's pieces are added in the order of their channels all the same
        for (int c0 = lane * 8; c0 < n; c0 += 256 * DEEP) {
            uint4 raw[DEEP][R];
#pragma unroll
            for (int d = 0; d < DEEP; ++d)
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (c0 + d * 256 < n) raw[d][r] = *reinterpret_cast<const uint4*>(w[r] + c0 + d * 256);
#pragma unroll
            for (int d = 0; d < DEEP; ++d) {
                const int c = c0 + d * 256;
                if (c >= n) break;
#pragma unroll
                for (int g = 0; g < R / XG; ++g) {
                    const float4 x0 = *reinterpret_cast<const float4*>(xs[g] + c), x1 = *reinterpret_cast<const float4*>(xs[g] + c + 4);
                    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int q = 0; q < XG; ++q) {
                        const int r = g * XG + q;
                        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[d][r]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(p[i]);
                            a[r] = fmaf(f.x, xv[2 * i], a[r]);
                            a[r] = fmaf(f.y, xv[2 * i + 1], a[r]);
                        }
                    }
                }
            }
        }
        return;
    }
    for (int c = lane; c < n; c += 32) {
#pragma unroll
        for (int r = 0; r < R; ++r) a[r] = fmaf(forge::to_float(w[r][c]), xs[r / XG][c], a[r]);
    }
}

// grid (pairs, ceil(F / 16)): act[pair, j] = act_fn(Wg[e][j] . x) * (Wu[e][j] . x);  row j of expert e lies at (e * F + j) * ld
// in both (ld = W: two matrices [E, F, W]; ld = 2 W and Wu = Wg + W: one matrix whose rows alternate gate, up).
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
moe_pair_gate_up_kernel(const TA* __restrict__ x, const TW* __restrict__ Wg, const TW* __restrict__ Wu, const int32_t* __restrict__ idx,
                        TA* __restrict__ act, int W, int F, int top, long long ld) {
    extern __shared__ __align__(16) float xs[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int p = blockIdx.x, t = p / top, e = idx[p];
    for (int c = threadIdx.x; c < W; c += 128) xs[c] = forge::to_float(x[(size_t)t * W + c]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j0 = blockIdx.y * kPairTile + warp * 4;
    if (j0 >= F) return;
    const TW* rows[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const size_t row = ((size_t)e * F + min(j0 + q, F - 1)) * ld;      // beyond the last output: its row once more, not written
        rows[2 * q] = Wg + row;
        rows[2 * q + 1] = Wu + row;
    }
    const float* const xv[1] = {xs};
    float a[8];
    lane_dot_rows<TW, 8, 8>(rows, xv, W, lane, a);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float g = forge::warp_sum(a[2 * q]), u = forge::warp_sum(a[2 * q + 1]);
        if (lane == 0 && j0 + q < F) act[(size_t)p * F + j0 + q] = forge::from_float<TA>(siluf(g) * u);
    }
}

// grid (T, ceil(Wd / 16)): y[t, n] = sum_k wts[t, k] * (Wd[e_k][n] . act[(t, k)]);  Wd [E, W, F].
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
moe_pair_down_kernel(const TA* __restrict__ act, const TW* __restrict__ Wd, const int32_t* __restrict__ idx, const float* __restrict__ wts,
                     float* __restrict__ y, int W, int F, int top) {
    extern __shared__ __align__(16) float as[];             // [top][F]
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * F; i += 128) as[i] = forge::to_float(act[(size_t)t * top * F + i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * kPairTile + warp * 4;
    if (n0 >= W) return;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    // two of the token's experts at a time (the last one alone if their number is odd), added in the router's order
    for (int k = 0; k < top; k += 2) {
        const int k1 = min(k + 1, top - 1);
        const int e0 = idx[(size_t)t * top + k], e1 = idx[(size_t)t * top + k1];
        const TW* rows[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int n = min(n0 + q, W - 1);
            rows[q] = Wd + ((size_t)e0 * W + n) * F;
            rows[4 + q] = Wd + ((size_t)e1 * W + n) * F;
        }
        const float* const av[2] = {as + (size_t)k * F, as + (size_t)k1 * F};
        float d[8];
        lane_dot_rows<TW, 8, 4, 2>(rows, av, F, lane, d);
        const float w0 = wts[(size_t)t * top + k], w1 = wts[(size_t)t * top + k1];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            sum[q] = fmaf(w0, forge::warp_sum(d[q]), sum[q]);
            const float second = forge::warp_sum(d[4 + q]);
            if (k + 1 < top) sum[q] = fmaf(w1, second, sum[q]);
        }
    }
    if (lane == 0)
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (n0 + q < W) y[(size_t)t * W + n0 + q] = sum[q];
}

constexpr int kGroupTokens = 8;           // input rows that share one pass over an expert's weight rows

// The same sums as the two kernels above, expert by expert, so that a weight row is read once for up to 8 of the expert's
// pairs instead of once per pair: grid (E, ceil(N / 32)).  A CTA lists the pairs that chose its expert (in order), stages
// their input rows in shared memory eight at a time and gives every warp 8 of the 32 output rows.
//   GATED:  out[p, j] = act_fn(Wa[e][j] . in[p / in_div]) * (Wb[e][j] . in[p / in_div])   (out of the activations' type)
//   else:   out[p, j] = Wa[e][j] . in[p]                                                   (out fp32; a later kernel weighs and adds)
// Row j of expert e lies at e * expert_stride + j * ld.  A dot product is dealt to the lanes and summed exactly as lane_dot
// does, so a pair's numbers do not depend on which of the paths took it.
template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(128)
moe_expert_rows_kernel(const TA* __restrict__ in, int in_div, const TW* __restrict__ Wa, const TW* __restrict__ Wb, long long ld,
                       long long expert_stride, const int32_t* __restrict__ idx, void* __restrict__ out_, int P, int K, int N, int nt_max) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __shared__ int s_count;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    float* xs = reinterpret_cast<float*>(moe_smem);                        // [nt_max][K]
    int* plist = reinterpret_cast<int*>(xs + (size_t)nt_max * K);          // [P]
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {                                                       // the expert's pairs, in order
        int n = 0;
        for (int p0 = 0; p0 < P; p0 += 32) {
            const bool mine = p0 + lane < P && idx[p0 + lane] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) plist[n + __popc(m & ((1u << lane) - 1u))] = p0 + lane;
            n += __popc(m);
        }
        if (lane == 0) s_count = n;
    }
    __syncthreads();
    const int count = s_count;
    const TW* wa = Wa + (size_t)e * expert_stride;
    const TW* wb = GATED ? Wb + (size_t)e * expert_stride : nullptr;
    const bool vec = std::is_same<TW, __nv_bfloat16>::value && (K & 7) == 0 && (ld & 7) == 0 && (expert_stride & 7) == 0 &&
                     (((uintptr_t)Wa) & 15) == 0 && (!GATED || (((uintptr_t)Wb) & 15) == 0);
    for (int g0 = 0; g0 < count; g0 += nt_max) {
        const int nt = min(nt_max, count - g0);
        __syncthreads();                                                   // the group before is done with xs
        for (int i = threadIdx.x; i < nt * K; i += 128) {
            const int n = i / K, c = i - n * K;
            xs[i] = forge::to_float(in[(size_t)(plist[g0 + n] / in_div) * K + c]);
        }
        __syncthreads();
        for (int jj = 0; jj < kPairOutputs / 4; ++jj) {
            const int j = blockIdx.y * kPairOutputs + warp * (kPairOutputs / 4) + jj;
            if (j >= N) break;
            float a[kGroupTokens], b[kGroupTokens];
#pragma unroll
            for (int n = 0; n < kGroupTokens; ++n) a[n] = b[n] = 0.f;
            const TW* ra = wa + (size_t)j * ld;
            const TW* rb = GATED ? wb + (size_t)j * ld : nullptr;
            if (vec) {
                for (int c = lane * 8; c < K; c += 256) {
                    const uint4 raw_a = *reinterpret_cast<const uint4*>(ra + c);
                    uint4 raw_b = raw_a;
                    if (GATED) raw_b = *reinterpret_cast<const uint4*>(rb + c);
                    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&raw_a);
                    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw_b);
                    float fa[8], fb[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 u = __bfloat1622float2(pa[i]), v = __bfloat1622float2(pb[i]);
                        fa[2 * i] = u.x; fa[2 * i + 1] = u.y; fb[2 * i] = v.x; fb[2 * i + 1] = v.y;
                    }
#pragma unroll
                    for (int n = 0; n < kGroupTokens; ++n) {
                        if (n >= nt) break;
                        const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)n * K + c);
                        const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)n * K + c + 4);
                        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            a[n] = fmaf(fa[i], xv[i], a[n]);
                            if (GATED) b[n] = fmaf(fb[i], xv[i], b[n]);
                        }
                    }
                }
            } else {
                for (int c = lane; c < K; c += 32) {
                    const float fa = forge::to_float(ra[c]), fb = GATED ? forge::to_float(rb[c]) : 0.f;
#pragma unroll
                    for (int n = 0; n < kGroupTokens; ++n) {
                        if (n >= nt) break;
                        a[n] = fmaf(fa, xs[(size_t)n * K + c], a[n]);
                        if (GATED) b[n] = fmaf(fb, xs[(size_t)n * K + c], b[n]);
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < kGroupTokens; ++n) {
                if (n >= nt) break;
                const float sa = forge::warp_sum(a[n]);
                const float sb = GATED ? forge::warp_sum(b[n]) : 0.f;
                if (lane == 0) {
                    const size_t o = (size_t)plist[g0 + n] * N + j;
                    if (GATED) reinterpret_cast<TA*>(out_)[o] = forge::from_float<TA>(siluf(sa) * sb);
                    else reinterpret_cast<float*>(out_)[o] = sa;
                }
            }
        }
    }
}

// One CTA per expert walks all pairs in order: rank[p] = how many earlier pairs chose the same expert; counts[e].
__global__ void __launch_bounds__(256)
moe_rank_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ rank, int32_t* __restrict__ counts, int P) {
    __shared__ int warp_tot[8];
    __shared__ int base;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int p0 = 0; p0 < P; p0 += 256) {
        const int p = p0 + threadIdx.x;
        const bool mine = p < P && idx[p] == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_tot[warp] = __popc(m);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (mine) rank[p] = before + __popc(m & ((1u << lane) - 1u));
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < 8; ++w) tot += warp_tot[w];
            base += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base;
}

// One CTA per pair: its row in the sorted order = (pairs of lower experts) + rank, or with room for `cap` rows per expert
// (cap > 0) expert * cap + rank; copies the token's input there.
template <typename TA>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const TA* __restrict__ x, const int32_t* __restrict__ idx, const int32_t* __restrict__ rank,
                  const int32_t* __restrict__ counts, int32_t* __restrict__ dest, TA* __restrict__ xg, int W, int top, int cap) {
    __shared__ int s_dest;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int p = blockIdx.x, t = p / top;
    if (threadIdx.x == 0) {
        const int e = idx[p];
        int off = e * cap;
        if (cap <= 0)
            for (int i = 0; i < e; ++i) off += counts[i];
        s_dest = off + rank[p];
        dest[p] = s_dest;
    }
    __syncthreads();
    const TA* src = x + (size_t)t * W;
    TA* dst = xg + (size_t)s_dest * W;
    for (int c = threadIdx.x; c < W; c += 128) dst[c] = src[c];
}

// y[t, :] = sum_k wts[t, k] * ys[dest[t, k], :], k in order.
__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ ys, const int32_t* __restrict__ dest, const float* __restrict__ wts, float* __restrict__ y,
                   int W, int top) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    if ((W & 3) == 0 && (((uintptr_t)ys | (uintptr_t)y) & 15) == 0) {          // four channels a load, the experts in the same order
#pragma unroll 4
        for (int c = threadIdx.x * 4; c < W; c += 512) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float w = wts[(size_t)t * top + k];
                const float4 v = *reinterpret_cast<const float4*>(ys + (size_t)dest[(size_t)t * top + k] * W + c);
                sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
            }
            *reinterpret_cast<float4*>(y + (size_t)t * W + c) = sum;
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += 128) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) sum = fmaf(wts[(size_t)t * top + k], ys[(size_t)dest[(size_t)t * top + k] * W + c], sum);
        y[(size_t)t * W + c] = sum;
    }
}

}  // namespace

// x [T, W] of type dtype; Wr fp32 [E, W]; idx int32 [T, top]; wts fp32 [T, top].  softmax 0: scores are sigmoids.
// corr fp32 [E] or null; groups <= 1: no groups, else E % groups == 0 and 1 <= keep <= groups with top <= keep * E / groups.
extern "C" int forge_moe_route(const void* x, int dtype, const float* Wr, int32_t* idx, float* wts, int T, int W, int E, int top,
                               int softmax, int renorm, const float* corr, int groups, int keep, float factor, cudaStream_t stream) {
    if (T < 0 || W <= 0 || E <= 0 || top <= 0 || top > E) return forge::fail(FORGE_ERR_ARG, "moe_route: bad sizes T=%d W=%d E=%d top=%d", T, W, E, top);
    if (groups > 1 && (E % groups != 0 || keep < 1 || keep > groups || top > keep * (E / groups)))
        return forge::fail(FORGE_ERR_ARG, "moe_route: %d experts in %d groups of which %d are kept, %d experts a token", E, groups, keep, top);
    if (E > 2048) return forge::fail(FORGE_ERR_UNSUPPORTED, "moe_route: %d experts", E);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(moe_route_kernel<TT>, dim3(T), dim3(kRouteThreads), sizeof(float) * (2 * E + (groups > 1 ? groups : 0)), stream, 1, (const TT*)x, Wr,
                          idx, wts, T, W, E, top, softmax, renorm, corr, groups > 1 ? groups : 0, keep, factor));
    return forge::check_launch("moe_route", e);
}

// x [T, W], act [T*top, F] of type dtype; Wg, Wu of type dtype, row j of expert e at (e * F + j) * ld elements.
extern "C" int forge_moe_pair_gate_up(const void* x, const void* Wg, const void* Wu, const int32_t* idx, void* act, int dtype, int T,
                                      int W, int F, int top, long long ld, cudaStream_t stream) {
    if (T < 0 || W <= 0 || F <= 0 || top <= 0) return forge::fail(FORGE_ERR_ARG, "moe_pair_gate_up: bad sizes T=%d W=%d F=%d top=%d", T, W, F, top);
    if (W > 12000) return forge::fail(FORGE_ERR_UNSUPPORTED, "moe_pair_gate_up: rows of %d", W);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(moe_pair_gate_up_kernel<TT, TT>, dim3(T * top, (F + kPairTile - 1) / kPairTile), dim3(128), sizeof(float) * W,
                          stream, 1, (const TT*)x, (const TT*)Wg, (const TT*)Wu, idx, (TT*)act, W, F, top, ld));
    return forge::check_launch("moe_pair_gate_up", e);
}

// act [T*top, F] of type dtype; Wd [E, W, F] of type dtype; y fp32 [T, W].
extern "C" int forge_moe_pair_down(const void* act, const void* Wd, const int32_t* idx, const float* wts, float* y, int dtype, int T, int W,
                                   int F, int top, cudaStream_t stream) {
    if (T < 0 || W <= 0 || F <= 0 || top <= 0) return forge::fail(FORGE_ERR_ARG, "moe_pair_down: bad sizes T=%d W=%d F=%d top=%d", T, W, F, top);
    if ((size_t)top * F * sizeof(float) > 200 * 1024) return forge::fail(FORGE_ERR_UNSUPPORTED, "moe_pair_down: %d experts of %d channels a token", top, F);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    static forge::PerDeviceFlag attr[2];
    bool& done = attr[dtype == FORGE_BF16].current();
    if (!done && (size_t)top * F * sizeof(float) > 48 * 1024) {
        FORGE_DISPATCH_DTYPE(dtype, TT,
            e = cudaFuncSetAttribute(moe_pair_down_kernel<TT, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (e != cudaSuccess) return forge::check_launch("moe_pair_down (shared memory)", e);
        done = true;
    }
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(moe_pair_down_kernel<TT, TT>, dim3(T, (W + kPairTile - 1) / kPairTile), dim3(128), sizeof(float) * top * F, stream,
                          1, (const TT*)act, (const TT*)Wd, idx, wts, y, W, F, top));
    return forge::check_launch("moe_pair_down", e);
}

namespace {
constexpr size_t kExpertSmemLimit = 200 * 1024;
forge::PerDeviceFlag g_expert_attr[4];

// rows staged at a time for a reduction of K channels and P pairs, 0 if not even one fits
int expert_rows_group(int K, int P) {
    const size_t left = kExpertSmemLimit - std::min(kExpertSmemLimit, (size_t)P * sizeof(int));
    return (int)std::min<size_t>(kGroupTokens, left / ((size_t)K * sizeof(float)));
}

template <typename TT, bool GATED>
cudaError_t launch_expert_rows(int which, cudaStream_t stream, const void* in, int in_div, const void* Wa, const void* Wb, long long ld,
                               long long expert_stride, const int32_t* idx, void* out, int P, int K, int N, int E) {
    const int nt = expert_rows_group(K, P);
    const size_t smem = (size_t)nt * K * sizeof(float) + (size_t)P * sizeof(int);
    bool& done = g_expert_attr[which].current();
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(moe_expert_rows_kernel<TT, TT, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kExpertSmemLimit);
        if (e != cudaSuccess) return e;
        done = true;
    }
    return forge::launch(moe_expert_rows_kernel<TT, TT, GATED>, dim3(E, (N + kPairOutputs - 1) / kPairOutputs), dim3(128), smem, stream, 1,
                         (const TT*)in, in_div, (const TT*)Wa, (const TT*)Wb, ld, expert_stride, idx, out, P, K, N, nt);
}
}  // namespace

// 1 if the expert-by-expert path takes a step of P pairs with reductions of W and F channels.
extern "C" int forge_moe_expert_supports(int P, int W, int F) { return (expert_rows_group(W, P) >= 1 && expert_rows_group(F, P) >= 1) ? 1 : 0; }

// The path by pairs, expert by expert: act [P, F] of type dtype (scratch), ys fp32 [P, W] = W_down[e_p] act[p] (a later
// moe_combine with dest[p] = p weighs and adds).  x [T, W]; Wg, Wu as in forge_moe_pair_gate_up; Wd [E, W, F]; idx int32 [P = T * top].
extern "C" int forge_moe_expert_rows(const void* x, const void* Wg, const void* Wu, long long ld, const void* Wd, const int32_t* idx, void* act,
                                     float* ys, int dtype, int T, int W, int F, int E, int top, cudaStream_t stream) {
    if (T < 0 || W <= 0 || F <= 0 || E <= 0 || top <= 0) return forge::fail(FORGE_ERR_ARG, "moe_expert_rows: bad sizes T=%d W=%d F=%d E=%d top=%d", T, W, F, E, top);
    const int P = T * top;
    if (!forge_moe_expert_supports(P, W, F)) return forge::fail(FORGE_ERR_UNSUPPORTED, "moe_expert_rows: rows of %d and %d channels, %d pairs", W, F, P);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT, {
        e = launch_expert_rows<TT, true>(dtype == FORGE_BF16 ? 0 : 1, stream, x, top, Wg, Wu, ld, (long long)F * ld, idx, act, P, W, F, E);
        if (e == cudaSuccess)
            e = launch_expert_rows<TT, false>(dtype == FORGE_BF16 ? 2 : 3, stream, act, 1, Wd, nullptr, F, (long long)W * F, idx, ys, P, F, W, E);
    });
    return forge::check_launch("moe_expert_rows", e);
}

// idx int32 [P]; rank, dest int32 [P]; counts int32 [E]; x [T, W]; xg of type dtype: [P, W], or with cap > 0 [E * cap, W], expert e's
// rows from row e * cap on (cap >= the most pairs one expert can get; the rows beyond an expert's count are not written).
extern "C" int forge_moe_sort(const void* x, int dtype, const int32_t* idx, int32_t* rank, int32_t* counts, int32_t* dest, void* xg, int T,
                              int W, int E, int top, int cap, cudaStream_t stream) {
    if (T < 0 || W <= 0 || E <= 0 || top <= 0) return forge::fail(FORGE_ERR_ARG, "moe_sort: bad sizes T=%d W=%d E=%d top=%d", T, W, E, top);
    if (T == 0) return FORGE_OK;
    cudaError_t e = forge::launch(moe_rank_kernel, dim3(E), dim3(256), 0, stream, 1, idx, rank, counts, T * top);
    if (e != cudaSuccess) return forge::check_launch("moe_sort (rank)", e);
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(moe_gather_kernel<TT>, dim3(T * top), dim3(128), 0, stream, 1, (const TT*)x, idx, rank, counts, dest, (TT*)xg, W, top, cap));
    return forge::check_launch("moe_sort", e);
}

// ys fp32 [P, W] in sorted order; y fp32 [T, W].
extern "C" int forge_moe_combine(const float* ys, const int32_t* dest, const float* wts, float* y, int T, int W, int top, cudaStream_t stream) {
    if (T < 0 || W <= 0 || top <= 0) return forge::fail(FORGE_ERR_ARG, "moe_combine: bad sizes T=%d W=%d top=%d", T, W, top);
    if (T == 0) return FORGE_OK;
    cudaError_t e = forge::launch(moe_combine_kernel, dim3(T), dim3(128), 0, stream, 1, ys, dest, wts, y, W, top);
    return forge::check_launch("moe_combine", e);
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
