// Mixers that carry a matrix of state per head from token to token, and the small steps around them.
//
// A head has K key channels and K value channels; its state S is [K, K] (key channel x value channel) in fp32,
// one per request slot, and everything that enters the recurrence is fp32.  Two recurrences:
//
//   decay-and-bonus ("wkv"):   o_t = (S + diag(u) k_t v_t^T)^T r_t ;   S <- diag(w_t) S + k_t v_t^T
//                              w_t = exp(-exp(x_t + w0))
//   generalized delta rule:    S <- diag(w_t) S - (a_t * n_t) (n_t^T S) + k_t v_t^T ;   o_t = S^T r_t
//                              n_t = k_t / sqrt(|k_t|^2 + 1e-6),  w_t = exp(-exp(-1/2) sigmoid(x_t + w0)),
//                              a_t = sigmoid(y_t + a0)               (both terms read the state before the step)
//   gated write (HGRN2):       S <- diag(f_t) S + (1 - f_t) v_t^T ;   o_t = S^T q_t          (no key: the forget gate also
//                              f_t = l + (1 - l) sigmoid(x_t + b),  q_t = silu(y_t)            decides what is written)
//   retention:                 S <- g S + k_t v_t^T ;   o_t = S^T q_t                         (one fixed decay g per head; q and k
//                              rotated by their position, k times K^-1/2, by retention_prepare_kernel)
//
// In the last two the state is [K, V] with V value channels that need not equal K; the first two have V = K.
//
// A CTA per (request, head, 16 columns of S) walks the request's tokens of the step in order; column j of S (the K numbers
// that meet value channel j) lives in the registers of eight neighbouring threads, so a token costs K/8 multiply-adds per
// thread, three shuffles, and no other exchange between threads except the vectors r, k, w (, a) of the token, which are
// staged in shared memory a few tokens at a time.  The walk is the same whether a request's tokens come in one step or in many: state and sums
// see the same operations in the same order.
#include "common.cuh"

namespace {

constexpr int kScanTokens = 8;        // tokens whose vectors are staged at a time

struct ScanInput {                    // a [T, heads * K] fp32 matrix that may be a column slice of a wider one
    const float* p;
    int ld;
};

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

constexpr int kSplit = 8;             // threads that share a column of S (each holds an eighth of its rows)
constexpr int kCols = 16;             // columns of S per CTA
constexpr int kScanThreads = kSplit * kCols;

// What the recurrence multiplies with, made in place from what the projections gave, for all tokens at once, a warp per
// (token, head):   MODE 0: x <- exp(-exp(x + w0));
//                  MODE 1: x <- exp(-exp(-1/2) sigmoid(x + w0)),  y <- sigmoid(y + a0),  inv[t, head] = 1 / (|k|^2 + 1e-6)
//                  MODE 2: x <- a0 + (1 - a0) sigmoid(x + w0)  (a0: the gate's lower bound),  y <- y sigmoid(y)
template <int MODE>
__global__ void __launch_bounds__(128)
scan_gates_kernel(float* __restrict__ x, int ld_x, float* __restrict__ y, int ld_y, const float* __restrict__ k, int ld_k,
                  float* __restrict__ inv, const float* __restrict__ w0, const float* __restrict__ a0, int T, int N, int K) {
    // No early word to the scheduler here: the kernel that follows is the scan, whose few CTAs each walk a request's tokens
    // for the whole of its time.  Let in while this kernel's many blocks fill the SMs, they were placed wherever there was
    // room, several on one SM and none on others, and the delta rule's scan took 850 us instead of 290 (1,024 tokens, 32
    // heads of 64).  They are let in when this grid's blocks exit and the SMs are free.
    forge::pdl_wait();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= T * N) return;
    const size_t t = w / N;
    const int head = w % N;
    float kk = 0.f;
    for (int ch = lane; ch < K; ch += 32) {
        const int c = head * K + ch;
        float* px = x + t * ld_x + c;
        if (MODE == 0) {
            *px = expf(-expf(*px + w0[c]));
        } else if (MODE == 2) {
            const float low = a0[c];
            *px = low + (1.0f - low) * sigmoidf(*px + w0[c]);
            float* py = y + t * ld_y + c;
            *py = *py * sigmoidf(*py);
        } else {
            *px = expf(-0.6065306597126334f * sigmoidf(*px + w0[c]));
            float* py = y + t * ld_y + c;
            *py = sigmoidf(*py + a0[c]);
            const float kv = k[t * ld_k + c];
            kk = fmaf(kv, kv, kk);
        }
    }
    if (MODE == 1) {
        kk = forge::warp_sum(kk);
        if (lane == 0) inv[w] = 1.0f / (kk + 1e-6f);
    }
}

__device__ __forceinline__ void stage_async(float* dst, const float* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    if (bytes == 16) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// MODE 0: decay and bonus; MODE 1: generalized delta rule; MODE 2: gated write (no k: 1 - d stands for it; KV value
// channels, the columns of S).  d: the decays, a: the removal rates (MODE 1), both ready made
// (scan_gates_kernel).  last_in (MODE 0, may be null): the mixer's input rows [T, W] of the activation type; the
// request's last row is kept as fp32 at state + prev_off (the next step's "previous token").
//
// A CTA has 16 columns of one head's S; thread (jl, q) = (tid / 8, tid % 8) holds the rows (4m + e) with m % 8 == q of
// column blockIdx.z*16 + jl (so the eight threads of a column read neighbouring 16-byte pieces of a staged vector), a
// token is KMAX/8 multiply-adds deep per thread and the eight partial sums of a column meet by three shuffles, always
// in the same order.  A head's columns are spread over K/16 CTAs so that one long request keeps many SMs busy, each
// with one warp per scheduler.  The vectors of the next kScanTokens tokens are copied into the other half of the staging
// buffers (cp.async, no stop in registers) while the present ones are worked on.
template <int KMAX, int MODE, typename TA>
__global__ void __launch_bounds__(kScanThreads)
state_scan_kernel(ScanInput r, ScanInput k, ScanInput v, ScanInput d, ScanInput a, const float* __restrict__ bonus,
                  const float* __restrict__ inv, float* __restrict__ state, long long state_stride, const int32_t* __restrict__ q_start,
                  const int32_t* __restrict__ slots, float* __restrict__ out, const TA* __restrict__ last_in, int W,
                  long long prev_off, int N, int K, int KV, int vec) {
    constexpr int RPT = KMAX / kSplit;                                  // rows of S per thread
    __shared__ __align__(16) float rs[2][kScanTokens][KMAX], ks[2][MODE == 2 ? 1 : kScanTokens][KMAX], ds[2][MODE == 3 ? 1 : kScanTokens][KMAX];
    __shared__ __align__(16) float as[2][MODE == 1 ? kScanTokens : 1][KMAX], vs[2][kScanTokens][kCols], us[KMAX];
    __shared__ float is[2][kScanTokens];                                // MODE 1: 1 / (|k|^2 + 1e-6) of the staged tokens
    forge::pdl_launch_dependents();
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, jl = tid / kSplit, q = tid % kSplit;
    const int j = blockIdx.z * kCols + jl;
    const bool live = j < KV;
    const int col = head * KV + j;
    // channels beyond K stay zero in every staged vector: the copies never touch them
    for (int i = tid; i < 2 * kScanTokens * KMAX; i += kScanThreads) {
        (&rs[0][0][0])[i] = 0.f;
        if (MODE != 2) (&ks[0][0][0])[i] = 0.f;          // (mode 2 has no keys: its ks is a stub that nothing reads)
        if (MODE != 3) (&ds[0][0][0])[i] = 0.f;          // (mode 3 has one decay per head: nothing staged)
        if (MODE == 1) (&as[0][0][0])[i] = 0.f;
    }
    for (int i = tid; i < 2 * kScanTokens * kCols; i += kScanThreads) (&vs[0][0][0])[i] = 0.f;
    for (int i = tid; i < KMAX; i += kScanThreads) us[i] = (MODE == 0 && i < K) ? bonus[head * K + i] : 0.f;
    __syncthreads();
    forge::pdl_wait();
    const int t_lo = q_start[s], t_hi = q_start[s + 1];
    float* S_g = state + (size_t)slots[s] * state_stride + (size_t)head * K * KV;
    // row of S that this thread's register ii holds
    auto row_of = [&](int ii) { return ((ii >> 2) * kSplit + q) * 4 + (ii & 3); };
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = (live && row_of(ii) < K) ? S_g[(size_t)row_of(ii) * KV + j] : 0.f;

    const int piece = vec ? 4 : 1, pieces = K / piece;                   // a staged vector in pieces of 16 or 4 bytes
    auto fetch = [&](int buf, int tb) {
        const int n = min(kScanTokens, t_hi - tb);
        for (int p = tid; p < n * pieces; p += kScanThreads) {
            const int tt = p / pieces, ch = (p % pieces) * piece;
            const size_t t = (size_t)(tb + tt), c = (size_t)head * K + ch;
            stage_async(&rs[buf][tt][ch], r.p + t * r.ld + c, piece * 4);
            if (MODE != 2) stage_async(&ks[buf][tt][ch], k.p + t * k.ld + c, piece * 4);
            if (MODE != 3) stage_async(&ds[buf][tt][ch], d.p + t * d.ld + c, piece * 4);
            if (MODE == 1) stage_async(&as[buf][tt][ch], a.p + t * a.ld + c, piece * 4);
        }
        const int tt = tid / kCols, jc = blockIdx.z * kCols + tid % kCols;              // values: this CTA's columns only
        if (tt < n && jc < KV) stage_async(&vs[buf][tt][tid % kCols], v.p + (size_t)(tb + tt) * v.ld + head * KV + jc, 4);
        if (MODE == 1 && tid < n) stage_async(&is[buf][tid], inv + (size_t)(tb + tid) * N + head, 4);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const float head_decay = MODE == 3 ? d.p[head] : 0.f;       // mode 3: d is one number per head
    fetch(0, t_lo);
    int buf = 0;
    for (int tb = t_lo; tb < t_hi; tb += kScanTokens, buf ^= 1) {
        const int n = min(kScanTokens, t_hi - tb);
        if (tb + kScanTokens < t_hi) {
            fetch(buf ^ 1, tb + kScanTokens);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                                  // the group of tokens has landed for every thread
#pragma unroll 4
        for (int tt = 0; tt < n; ++tt) {
            const float vj = vs[buf][tt][jl];
            const float4* r4 = reinterpret_cast<const float4*>(&rs[buf][tt][0]) + q;
            const float4* k4 = reinterpret_cast<const float4*>(&ks[buf][tt][0]) + q;
            const float4* d4 = reinterpret_cast<const float4*>(&ds[buf][tt][0]) + q;
            float acc0 = 0.f, acc1 = 0.f;
            if (MODE == 0) {
                const float4* u4 = reinterpret_cast<const float4*>(&us[0]) + q;
#pragma unroll
                for (int c4 = 0; c4 < RPT / 4; ++c4) {
                    const float4 rr = r4[c4 * kSplit], kk = k4[c4 * kSplit], dd = d4[c4 * kSplit], uu = u4[c4 * kSplit];
                    const float rv[4] = {rr.x, rr.y, rr.z, rr.w}, kv4[4] = {kk.x, kk.y, kk.z, kk.w};
                    const float dv[4] = {dd.x, dd.y, dd.z, dd.w}, uv[4] = {uu.x, uu.y, uu.z, uu.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int ii = c4 * 4 + e;
                        const float kv = kv4[e] * vj;
                        if (e & 1) acc1 = fmaf(rv[e], fmaf(uv[e], kv, S[ii]), acc1);
                        else acc0 = fmaf(rv[e], fmaf(uv[e], kv, S[ii]), acc0);
                        S[ii] = fmaf(dv[e], S[ii], kv);
                    }
                }
            } else if (MODE == 3) {
#pragma unroll
                for (int c4 = 0; c4 < RPT / 4; ++c4) {
                    const float4 rr = r4[c4 * kSplit], kk = k4[c4 * kSplit];
                    const float rv[4] = {rr.x, rr.y, rr.z, rr.w}, kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int ii = c4 * 4 + e;
                        S[ii] = fmaf(head_decay, S[ii], kv4[e] * vj);
                        if (e & 1) acc1 = fmaf(rv[e], S[ii], acc1);
                        else acc0 = fmaf(rv[e], S[ii], acc0);
                    }
                }
            } else if (MODE == 2) {
#pragma unroll
                for (int c4 = 0; c4 < RPT / 4; ++c4) {
                    const float4 rr = r4[c4 * kSplit], dd = d4[c4 * kSplit];
                    const float rv[4] = {rr.x, rr.y, rr.z, rr.w}, dv[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int ii = c4 * 4 + e;
                        S[ii] = fmaf(dv[e], S[ii], (1.0f - dv[e]) * vj);
                        if (e & 1) acc1 = fmaf(rv[e], S[ii], acc1);
                        else acc0 = fmaf(rv[e], S[ii], acc0);
                    }
                }
            } else {
                const float4* a4 = reinterpret_cast<const float4*>(&as[buf][tt][0]) + q;
                float held0 = 0.f, held1 = 0.f;            // this thread's share of k^T S (its column)
#pragma unroll
                for (int c4 = 0; c4 < RPT / 4; ++c4) {
                    const float4 kk = k4[c4 * kSplit];
                    held0 = fmaf(kk.x, S[c4 * 4], held0);
                    held1 = fmaf(kk.y, S[c4 * 4 + 1], held1);
                    held0 = fmaf(kk.z, S[c4 * 4 + 2], held0);
                    held1 = fmaf(kk.w, S[c4 * 4 + 3], held1);
                }
                float held = held0 + held1;
#pragma unroll
                for (int o = 1; o < kSplit; o <<= 1) held += __shfl_xor_sync(0xffffffffu, held, o);
                // (a * n)(n^T S) = a_i k_i (k^T S) / (|k|^2 + 1e-6): the two roots of the unit key multiply out
                const float share = held * is[buf][tt];
#pragma unroll
                for (int c4 = 0; c4 < RPT / 4; ++c4) {
                    const float4 rr = r4[c4 * kSplit], kk = k4[c4 * kSplit], dd = d4[c4 * kSplit], aa = a4[c4 * kSplit];
                    const float rv[4] = {rr.x, rr.y, rr.z, rr.w}, kv4[4] = {kk.x, kk.y, kk.z, kk.w};
                    const float dv[4] = {dd.x, dd.y, dd.z, dd.w}, av[4] = {aa.x, aa.y, aa.z, aa.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int ii = c4 * 4 + e;
                        S[ii] = fmaf(dv[e], S[ii], kv4[e] * (vj - av[e] * share));
                        if (e & 1) acc1 = fmaf(rv[e], S[ii], acc1);
                        else acc0 = fmaf(rv[e], S[ii], acc0);
                    }
                }
            }
            float acc = acc0 + acc1;
#pragma unroll
            for (int o = 1; o < kSplit; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && q == 0) out[(size_t)(tb + tt) * N * KV + col] = acc;
        }
        __syncthreads();                                                  // before the next copies overwrite this half
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii)
            if (row_of(ii) < K) S_g[(size_t)row_of(ii) * KV + j] = S[ii];
    }
    if (MODE == 0 && last_in != nullptr && t_hi > t_lo) {
        float* prev = state + (size_t)slots[s] * state_stride + prev_off;
        const TA* row = last_in + (size_t)(t_hi - 1) * W;
        const int ctas = N * gridDim.z;
        for (int c = (head * gridDim.z + blockIdx.z) * kScanThreads + tid; c < W; c += ctas * kScanThreads) prev[c] = forge::to_float(row[c]);
    }
}

// The shifted inputs of a mixer that looks one token back: out[m][t][c] = h[t][c] + (prev[t][c] - h[t][c]) * mu[m][c],
// prev = h[t-1] inside a request's tokens of the step, the kept row of the request's state for its first token.
template <typename TA>
__global__ void __launch_bounds__(128)
token_shift_kernel(const TA* __restrict__ h, const float* __restrict__ state, long long state_stride, long long prev_off,
                   const int32_t* __restrict__ tok_req, const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots,
                   const float* __restrict__ mu, TA* __restrict__ out, int T, int W, int n_mix) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x, s = tok_req[t];
    const bool first = t == q_start[s];
    const float* kept = state + (size_t)slots[s] * state_stride + prev_off;
    // (a step of few tokens spreads a row over several CTAs: a thread's loads are a chain, and eight CTAs walking 2,048
    // columns took 26 us)
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        const float cur = forge::to_float(h[(size_t)t * W + c]);
        const float prev = first ? kept[c] : forge::to_float(h[(size_t)(t - 1) * W + c]);
        for (int m = 0; m < n_mix; ++m)
            out[((size_t)m * T + t) * W + c] = forge::from_float<TA>(fmaf(prev - cur, mu[(size_t)m * W + c], cur));
    }
}

// One warp per (token, head): the head's K outputs divided by their root mean square, times a weight per channel,
// times a gate (act 0: sigmoid(g), 1: g * sigmoid(g), 2: no gate) and a number, stored in the activation type for the
// output projection.  share_w: the K weights are shared by the heads.
template <typename TA>
__global__ void __launch_bounds__(128)
head_finish_kernel(const float* __restrict__ o, const float* __restrict__ weight, ScanInput g, TA* __restrict__ out, int rows,
                   int N, int K, float eps, int act, float scale, int share_w, long long out_ld) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * N) return;
    const int t = w / N, head = w % N;
    const float* src = o + (size_t)t * N * K + head * K;
    float ss = 0.f;
    for (int c = lane; c < K; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = forge::warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)K + eps);
    for (int c = lane; c < K; c += 32) {
        float gate = scale;
        if (act != 2) {
            const float gv = g.p[(size_t)t * g.ld + head * K + c];
            gate = scale * (act == 1 ? gv * sigmoidf(gv) : sigmoidf(gv));
        }
        out[(size_t)t * out_ld + head * K + c] = forge::from_float<TA>(src[c] * inv * weight[share_w ? c : head * K + c] * gate);
    }
}

// out[t][c] = tanh(in[t][c]) in the activation type (the hidden layer of a low-rank projection).
template <typename TA>
__global__ void tanh_rows_kernel(ScanInput in, TA* __restrict__ out, int T, int n) {
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * n) return;
    out[i] = forge::from_float<TA>(tanhf(in.p[(i / n) * in.ld + i % n]));
}

// Retention's q and k on their way into the recurrence, in place, a warp per (token, head): the first rot_dims channels of
// both turn by position * freq (channel i paired with i + rot_dims/2), then k is multiplied by k_scale.
__global__ void __launch_bounds__(128)
retention_prepare_kernel(float* __restrict__ q, int ld_q, float* __restrict__ k, int ld_k, const int32_t* __restrict__ positions,
                         const float* __restrict__ freq, int rot_dims, float k_scale, int T, int N, int K) {
    forge::pdl_wait();             // (no early word: the scan follows, see scan_gates_kernel)
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= T * N) return;
    const size_t t = w / N;
    const int head = w % N, half = rot_dims >> 1;
    const float pos = (float)positions[t];
    float* qh = q + t * ld_q + head * K;
    float* kh = k + t * ld_k + head * K;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        const float qu = qh[i], qv = qh[i + half], ku = kh[i], kv = kh[i + half];
        qh[i] = qu * cs - qv * sn;
        qh[i + half] = qv * cs + qu * sn;
        kh[i] = (ku * cs - kv * sn) * k_scale;
        kh[i + half] = (kv * cs + ku * sn) * k_scale;
    }
    for (int c = rot_dims + lane; c < K; c += 32) kh[c] *= k_scale;
}

template <int MODE, typename TA>
cudaError_t launch_scan(int kmax, dim3 grid, cudaStream_t stream, ScanInput r, ScanInput k, ScanInput v, ScanInput d, ScanInput a,
                        const float* bonus, const float* inv, float* state, long long stride, const int32_t* q_start, const int32_t* slots,
                        float* out, const TA* last_in, int W, long long prev_off, int N, int K, int KV, int vec) {
#define FORGE_SCAN_CASE(KM)                                                                                                  \
    case KM:                                                                                                                 \
        return forge::launch(state_scan_kernel<KM, MODE, TA>, grid, dim3(kScanThreads), 0, stream, 1, r, k, v, d, a, bonus, inv, state, \
                             stride, q_start, slots, out, last_in, W, prev_off, N, K, KV, vec);
    if constexpr (MODE == 2 || MODE == 3) {   // the gated write stages no keys, retention no decays: heads of up to 256 key channels fit
        switch (kmax) {
            FORGE_SCAN_CASE(192) FORGE_SCAN_CASE(256)
            default: break;
        }
    }
    switch (kmax) {
        FORGE_SCAN_CASE(32) FORGE_SCAN_CASE(64) FORGE_SCAN_CASE(96) FORGE_SCAN_CASE(128)
        default: return cudaErrorInvalidValue;
    }
#undef FORGE_SCAN_CASE
}

}  // namespace

// mode 0 (decay and bonus) / 1 (generalized delta rule) / 2 (gated write: no k; x the forget gate's input with w0 its bias
// and a0 its lower bound; y = r, which becomes silu(r) in place; v and out have N*KV columns, a head's state is [K, KV]).
// KV = K in modes 0 and 1.  r, k, v, x (and y, mode 1): fp32, row t at p + t * ld, head n's
// channels at columns n*K .. n*K+K-1; x (and y) are OVERWRITTEN with the decays (and removal rates) made from them; T: rows
// of these matrices.  w0 (, a0, mode 1; bonus, mode 0): fp32 [N*K].  inv (mode 1): fp32 [T, N] scratch for 1 / (|k|^2 + 1e-6).  state: fp32 rows of state_stride
// numbers, row slots[s] holds request s's N matrices [K, K] from its start.  out fp32 [T, N*K].  last_in (mode 0, optional):
// the mixer's input [T, W] of type last_dtype, whose last row per request is kept at state + prev_off.
extern "C" int forge_state_scan(int mode, const float* r, int ld_r, const float* k, int ld_k, const float* v, int ld_v,
                                const float* x, int ld_x, const float* y, int ld_y, const float* w0, const float* a0,
                                const float* bonus, float* inv, float* state, long long state_stride, const int32_t* q_start,
                                const int32_t* slots, float* out, const void* last_in, int last_dtype, int W, long long prev_off,
                                int T, int S, int N, int K, int KV, cudaStream_t stream) {
    if (T < 0 || S < 0 || N <= 0 || K <= 0 || KV <= 0 || mode < 0 || mode > 2 || (mode != 2 && KV != K))
        return forge::fail(FORGE_ERR_ARG, "state_scan: bad sizes S=%d N=%d K=%d mode=%d", S, N, K, mode);
    if (K > (mode == 2 ? 256 : 128)) return forge::fail(FORGE_ERR_UNSUPPORTED, "state_scan: heads of %d channels (at most %d)", K, mode == 2 ? 256 : 128);
    if (state_stride < (long long)N * K * KV) return forge::fail(FORGE_ERR_ARG, "state_scan: state rows are too short");
    if (mode == 0 && !bonus) return forge::fail(FORGE_ERR_ARG, "state_scan: mode 0 needs the bonus");
    if (mode == 1 && (!y || !a0)) return forge::fail(FORGE_ERR_ARG, "state_scan: mode 1 needs the removal rate");
    if (mode == 2 && (y != r || ld_y != ld_r || !a0)) return forge::fail(FORGE_ERR_ARG, "state_scan: mode 2 takes y = r and the gate's lower bound");
    if (S == 0) return FORGE_OK;
    const int kmax = K <= 128 ? (K + 31) / 32 * 32 : (K <= 192 ? 192 : 256);
    const dim3 grid(S, N, (KV + kCols - 1) / kCols);
    // decays (and removal rates, and the unit keys' divisors) for all tokens at once, in place
    {
        if (mode == 1 && !inv) return forge::fail(FORGE_ERR_ARG, "state_scan: mode 1 needs room for the keys' divisors");
        const unsigned blocks = (unsigned)(((size_t)T * N + 3) / 4);
        cudaError_t g = mode == 2
            ? forge::launch(scan_gates_kernel<2>, dim3(blocks), dim3(128), 0, stream, 1, const_cast<float*>(x), ld_x, const_cast<float*>(y), ld_y,
                            (const float*)nullptr, 0, (float*)nullptr, w0, a0, T, N, K)
            : mode == 0
            ? forge::launch(scan_gates_kernel<0>, dim3(blocks), dim3(128), 0, stream, 1, const_cast<float*>(x), ld_x, (float*)nullptr, 0,
                            (const float*)nullptr, 0, (float*)nullptr, w0, a0, T, N, K)
            : forge::launch(scan_gates_kernel<1>, dim3(blocks), dim3(128), 0, stream, 1, const_cast<float*>(x), ld_x, const_cast<float*>(y), ld_y,
                            k, ld_k, inv, w0, a0, T, N, K);
        if (g != cudaSuccess) return forge::check_launch("state_scan (gates)", g);
    }
    ScanInput R{r, ld_r}, Kk{k, ld_k}, V{v, ld_v}, X{x, ld_x}, Y{y, ld_y};
    auto aligned = [](const float* p, int ld) { return p == nullptr || (((uintptr_t)p & 15) == 0 && ld % 4 == 0); };
    const int vec = (K % 4 == 0 && aligned(r, ld_r) && aligned(k, ld_k) && aligned(x, ld_x) && aligned(y, ld_y)) ? 1 : 0;
    cudaError_t e;
    if (mode == 2) {
        e = launch_scan<2, float>(kmax, grid, stream, R, R, V, X, Y, nullptr, nullptr, state, state_stride, q_start, slots, out, nullptr, 0, 0, N, K, KV, vec);
    } else if (mode == 1) {
        e = launch_scan<1, float>(kmax, grid, stream, R, Kk, V, X, Y, nullptr, inv, state, state_stride, q_start, slots, out, nullptr, 0, 0, N, K, K, vec);
    } else if (last_in == nullptr || last_dtype == FORGE_F32) {
        e = launch_scan<0, float>(kmax, grid, stream, R, Kk, V, X, Y, bonus, nullptr, state, state_stride, q_start, slots, out,
                                  (const float*)last_in, W, prev_off, N, K, K, vec);
    } else {
        e = launch_scan<0, __nv_bfloat16>(kmax, grid, stream, R, Kk, V, X, Y, bonus, nullptr, state, state_stride, q_start, slots, out,
                                          (const __nv_bfloat16*)last_in, W, prev_off, N, K, K, vec);
    }
    return forge::check_launch("state_scan", e);
}

// Retention over the step's tokens: q, k fp32 (row t at p + t * ld, head n's K channels at columns n*K ..) are rotated and
// scaled IN PLACE, then S <- decay[n] S + k v^T, out = S^T q per head; v and out have N*KV columns, a head's state is [K, KV].
// freq fp32 [rot_dims / 2] (null with rot_dims 0); decay fp32 [N].
extern "C" int forge_retention_scan(float* q, int ld_q, float* k, int ld_k, const float* v, int ld_v, const int32_t* positions,
                                    const float* freq, int rot_dims, float k_scale, const float* decay, float* state,
                                    long long state_stride, const int32_t* q_start, const int32_t* slots, float* out, int T, int S,
                                    int N, int K, int KV, cudaStream_t stream) {
    if (T < 0 || S < 0 || N <= 0 || K <= 0 || KV <= 0 || rot_dims < 0 || rot_dims > K || (rot_dims & 1))
        return forge::fail(FORGE_ERR_ARG, "retention_scan: bad sizes S=%d N=%d K=%d V=%d rot=%d", S, N, K, KV, rot_dims);
    if (K > 256) return forge::fail(FORGE_ERR_UNSUPPORTED, "retention_scan: heads of %d key channels (at most 256)", K);
    if (state_stride < (long long)N * K * KV) return forge::fail(FORGE_ERR_ARG, "retention_scan: state rows are too short");
    if (rot_dims > 0 && !freq) return forge::fail(FORGE_ERR_ARG, "retention_scan: a rotation needs its frequencies");
    if (S == 0 || T == 0) return FORGE_OK;
    const unsigned blocks = (unsigned)(((size_t)T * N + 3) / 4);
    cudaError_t e = forge::launch(retention_prepare_kernel, dim3(blocks), dim3(128), 0, stream, 1, q, ld_q, k, ld_k, positions, freq, rot_dims,
                                  k_scale, T, N, K);
    if (e != cudaSuccess) return forge::check_launch("retention_scan (prepare)", e);
    const int kmax = K <= 128 ? (K + 31) / 32 * 32 : (K <= 192 ? 192 : 256);
    const dim3 grid(S, N, (KV + kCols - 1) / kCols);
    ScanInput Q{q, ld_q}, Kk{k, ld_k}, V{v, ld_v}, D{decay, 0};
    auto aligned = [](const float* p, int ld) { return ((uintptr_t)p & 15) == 0 && ld % 4 == 0; };
    const int vec = (K % 4 == 0 && aligned(q, ld_q) && aligned(k, ld_k)) ? 1 : 0;
    e = launch_scan<3, float>(kmax, grid, stream, Q, Kk, V, D, D, nullptr, nullptr, state, state_stride, q_start, slots, out, nullptr, 0, 0,
                              N, K, KV, vec);
    return forge::check_launch("retention_scan", e);
}

// h, out of type dtype: [T, W] and [n_mix, T, W]; mu fp32 [n_mix, W]; the kept row of request s: state + slots[s] * stride + prev_off.
extern "C" int forge_token_shift(const void* h, const float* state, long long state_stride, long long prev_off, const int32_t* tok_req,
                                 const int32_t* q_start, const int32_t* slots, const float* mu, void* out, int dtype, int T, int W,
                                 int n_mix, cudaStream_t stream) {
    if (T < 0 || W <= 0 || n_mix <= 0) return forge::fail(FORGE_ERR_ARG, "token_shift: bad sizes T=%d W=%d n=%d", T, W, n_mix);
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(token_shift_kernel<TT>, dim3(T, T >= 256 ? 1 : (W + 511) / 512), dim3(128), 0, stream, 1, (const TT*)h, state, state_stride, prev_off, tok_req,
                          q_start, slots, mu, (TT*)out, T, W, n_mix));
    return forge::check_launch("token_shift", e);
}

// o fp32 [T, N*K]; weight fp32 [N*K]; g fp32 rows of ld_g (the gate before its activation); out of type dtype, rows of out_ld
// elements with the N*K values at their start.
extern "C" int forge_head_finish(const float* o, const float* weight, const float* g, int ld_g, void* out, int dtype, int T, int N,
                                 int K, float eps, int act, float scale, int share_w, long long out_ld, cudaStream_t stream) {
    if (out_ld < (long long)N * K) return forge::fail(FORGE_ERR_ARG, "head_finish: output rows of %lld are too short", out_ld);
    if (T < 0 || N <= 0 || K <= 0 || act < 0 || act > 2 || (act != 2 && !g)) return forge::fail(FORGE_ERR_ARG, "head_finish: bad sizes T=%d N=%d K=%d", T, N, K);
    if (T == 0) return FORGE_OK;
    if ((long long)T * N > 0x7fffffffLL / 2) return forge::fail(FORGE_ERR_UNSUPPORTED, "head_finish: too many rows");
    const unsigned blocks = (unsigned)(((long long)T * N + 3) / 4);
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(head_finish_kernel<TT>, dim3(blocks), dim3(128), 0, stream, 1, o, weight, ScanInput{g, ld_g}, (TT*)out, T, N, K,
                          eps, act, scale, share_w, out_ld));
    return forge::check_launch("head_finish", e);
}

extern "C" int forge_tanh_rows(const float* in, int ld, void* out, int dtype, int T, int n, cudaStream_t stream) {
    if (T < 0 || n <= 0 || ld < n) return forge::fail(FORGE_ERR_ARG, "tanh_rows: bad sizes T=%d n=%d ld=%d", T, n, ld);
    if (T == 0) return FORGE_OK;
    const unsigned blocks = (unsigned)(((size_t)T * n + 255) / 256);
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(tanh_rows_kernel<TT>, dim3(blocks), dim3(256), 0, stream, 1, ScanInput{in, ld}, (TT*)out, T, n));
    return forge::check_launch("tanh_rows", e);
}

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
