// Attention whose keys and values are made from one small latent vector per token, and the steps around it.
//
// A token leaves in the cache one row [c | kr]: the normed latent c (C channels) and one rotated key part kr (R channels)
// that all heads share.  Head h's key is [Wk_h c | kr] and its value Wv_h c, so with the query q_h = [qf | qr]
//     score(i, j) = scale (qf_i . Wk_h c_j + qr_i . kr_j) = scale [Wk_h^T qf_i | qr_i] . [c_j | kr_j]
//     o_i         = Wv_h sum_j p_ij c_j
// and the per-head matrices move to the query and to the output: every head attends with a query of C + R channels over the
// SAME rows (one key/value head for all query heads), values are a row's first C channels, and Wv_h is applied once per
// token afterwards.  Keys and values per head are never formed.
//
//   latent_prepare     the RMS norms of the two down-projections, the rotation of kr, the cache write
//   head_linear        out[t, h, :] = W_h^T in[t, h, :] for every head (W_h stored [K, N]), optionally followed by R more
//                      input channels that are rotated and copied behind the N outputs (the absorbed query)
//   latent_attention   causal softmax attention over the latent rows, fp32 arithmetic whatever the storage type
//
// The rotation pairs channel 2i with 2i + 1 and turns the pair by position * freq[i]; cos and sin are multiplied by `amp`.
// Keys are walked in chunks of KT positions that start at multiples of KT, a chunk's weights are summed in a fixed order,
// and a key that a token does not see adds exact zeros: what a token adds up, and in which order, depends on its position
// alone, not on the step's cut, the tile, or the batch around it.
#include "common.cuh"
#include "checks.cuh"
#include "mma_sync.cuh"

namespace {

constexpr int kPrepThreads = 128;

// One CTA per token.  proj fp32 row = [dq: Cq | c: C | kr: R] (C = 0: a layer that reads another layer's rows and has only dq).
template <typename TC>
__global__ void __launch_bounds__(kPrepThreads)
latent_prepare_kernel(const float* __restrict__ proj, int ld, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ slot_mapping, const float* __restrict__ freq, float amp,
                      const float* __restrict__ wq, const float* __restrict__ wc, TC* __restrict__ cq_out, TC* __restrict__ cache,
                      int Cq, int C, int R, float eps) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Cq; i += kPrepThreads) ss = fmaf(row[i], row[i], ss);
    const float inv_q = 1.0f / sqrtf(forge::block_sum(ss, red) / (float)Cq + eps);
    for (int i = threadIdx.x; i < Cq; i += kPrepThreads) cq_out[(size_t)t * Cq + i] = forge::from_float<TC>(row[i] * inv_q * wq[i]);
    if (C == 0 || slot_mapping == nullptr) return;
    const int slot = slot_mapping[t];
    if (slot < 0 || !FORGE_SLOT_OK(slot)) return;
    const float* c = row + Cq;
    ss = 0.f;
    for (int i = threadIdx.x; i < C; i += kPrepThreads) ss = fmaf(c[i], c[i], ss);
    const float inv_c = 1.0f / sqrtf(forge::block_sum(ss, red) / (float)C + eps);
    TC* dst = cache + (size_t)slot * (C + R);
    for (int i = threadIdx.x; i < C; i += kPrepThreads) dst[i] = forge::from_float<TC>(c[i] * inv_c * wc[i]);
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < (R >> 1); i += kPrepThreads) {
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= amp;
        cs *= amp;
        const float u = c[C + 2 * i], v = c[C + 2 * i + 1];
        dst[C + 2 * i] = forge::from_float<TC>(u * cs - v * sn);
        dst[C + 2 * i + 1] = forge::from_float<TC>(v * cs + u * sn);
    }
}

constexpr int kLinThreads = 128, kLinTokens = 8;

// One CTA per (8 tokens, head, 128 output channels).  in: row t, head h at in + t * in_ld + h * in_hs (K channels, then R
// channels to rotate); W [H, K, N]; out: row t, head h at out + t * out_ld + h * out_hs (N channels, then the R rotated).
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(kLinThreads)
head_linear_kernel(const TI* __restrict__ in, long long in_ld, int in_hs, const TW* __restrict__ W, TO* __restrict__ out,
                   long long out_ld, int out_hs, const int32_t* __restrict__ positions, const float* __restrict__ freq, float amp,
                   int T, int K, int N, int R, const float* __restrict__ gate, long long gate_ld) {
    extern __shared__ float xs[];                       // [kLinTokens][K]
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t0 = blockIdx.x * kLinTokens, h = blockIdx.y, nt = min(kLinTokens, T - t0);
    for (int i = threadIdx.x; i < kLinTokens * K; i += kLinThreads) {
        const int tt = i / K, k = i % K;
        xs[i] = tt < nt ? forge::to_float(in[(size_t)(t0 + tt) * in_ld + (size_t)h * in_hs + k]) : 0.f;
    }
    __syncthreads();
    const int n = blockIdx.z * kLinThreads + threadIdx.x;
    if (n < N) {
        float acc[kLinTokens];
#pragma unroll
        for (int tt = 0; tt < kLinTokens; ++tt) acc[tt] = 0.f;
        const TW* w = W + (size_t)h * K * N + n;
        for (int k = 0; k < K; ++k) {
            const float wv = forge::to_float(w[(size_t)k * N]);
#pragma unroll
            for (int tt = 0; tt < kLinTokens; ++tt) acc[tt] = fmaf(xs[tt * K + k], wv, acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < kLinTokens; ++tt)
            if (tt < nt) {
                float v = acc[tt];
                if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)(t0 + tt) * gate_ld + (size_t)h * N + n]));
                out[(size_t)(t0 + tt) * out_ld + (size_t)h * out_hs + n] = forge::from_float<TO>(v);
            }
    }
    if (R > 0 && blockIdx.z == 0) {
        for (int i = threadIdx.x; i < nt * (R >> 1); i += kLinThreads) {
            const int tt = i / (R >> 1), p = i % (R >> 1);
            const TI* src = in + (size_t)(t0 + tt) * in_ld + (size_t)h * in_hs + K;
            float sn, cs;
            sincosf((float)positions[t0 + tt] * freq[p], &sn, &cs);
            sn *= amp;
            cs *= amp;
            const float u = forge::to_float(src[2 * p]), v = forge::to_float(src[2 * p + 1]);
            TO* dst = out + (size_t)(t0 + tt) * out_ld + (size_t)h * out_hs + N;
            dst[2 * p] = forge::from_float<TO>(u * cs - v * sn);
            dst[2 * p + 1] = forge::from_float<TO>(v * cs + u * sn);
        }
    }
}

// The same per-head product on the tensor cores for 16-bit weights: one CTA of four warps per (64 tokens, head, 64 output
// channels), a warp 16 tokens.  The reduction runs over chunks of 128 input channels (all of a chunk's loads in flight at once); a chunk of the inputs (rounded to bfloat16
// where they come as fp32) and of W_h is staged in shared memory, rows padded by 16 bytes so that the 8 x 8 matrix loads do not
// meet in a bank, and multiplied by m16n8k16 products with fp32 sums.  Rows and channels beyond T, K and N are staged as
// zeros.  The rotated channels are taken by the CTAs of the first channel tile, as in the kernel above.
constexpr int kHlmThreads = 128, kHlmTile = 64, kHlmRow = kHlmTile + 8, kHlmK = 128, kHlmRowK = kHlmK + 8;

template <typename TI>
__device__ __forceinline__ uint4 load8_bf16(const TI* __restrict__ p, int valid, bool vec);
template <>
__device__ __forceinline__ uint4 load8_bf16<float>(const float* __restrict__ p, int valid, bool vec) {
    float f[8];
    if (vec && valid >= 8) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = i < valid ? p[i] : 0.f;
    }
    return make_uint4(mma_sync::pack_bf16(f[0], f[1]), mma_sync::pack_bf16(f[2], f[3]), mma_sync::pack_bf16(f[4], f[5]), mma_sync::pack_bf16(f[6], f[7]));
}
template <>
__device__ __forceinline__ uint4 load8_bf16<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, int valid, bool vec) {
    if (vec && valid >= 8) return *reinterpret_cast<const uint4*>(p);
    __align__(16) __nv_bfloat16 h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = i < valid ? p[i] : __float2bfloat16(0.f);
    return *reinterpret_cast<const uint4*>(h);
}

template <typename TI>
__global__ void __launch_bounds__(kHlmThreads)
head_linear_mma_kernel(const TI* __restrict__ in, long long in_ld, int in_hs, const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ out,
                       long long out_ld, int out_hs, const int32_t* __restrict__ positions, const float* __restrict__ freq, float amp,
                       int T, int K, int N, int R, const float* __restrict__ gate, long long gate_ld) {
    __shared__ __align__(16) __nv_bfloat16 As[kHlmTile][kHlmRowK];         // [token][input channel of the chunk]
    __shared__ __align__(16) __nv_bfloat16 Bs[kHlmK][kHlmRow];             // [input channel of the chunk][output channel]
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t0 = blockIdx.x * kHlmTile, h = blockIdx.y, n0 = blockIdx.z * kHlmTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kIn = 16 / (int)sizeof(TI);                              // input elements per 16 bytes
    const bool a_vec = (in_ld % kIn) == 0 && (in_hs % kIn) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0;
    const bool b_vec = (N & 7) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
    const __nv_bfloat16* Wh = W + (size_t)h * K * N;
    const int nt = min(kHlmTile, T - t0);
    const bool warp_live = warp * 16 < nt;                                 // a warp whose 16 tokens lie beyond the step's has no sums
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    constexpr int kPer = kHlmTile * kHlmK / 8 / kHlmThreads;               // 16-byte pieces per thread of each operand's chunk
    for (int k0 = 0; k0 < K; k0 += kHlmK) {
        uint4 av[kPer], bv[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = threadIdx.x + j * kHlmThreads;
            const int ra = i / (kHlmK / 8), ca = (i % (kHlmK / 8)) * 8;    // a token's piece of 8 input channels
            const int t = t0 + ra, k = k0 + ca;
            av[j] = make_uint4(0u, 0u, 0u, 0u);
            if (t < T && k < K) av[j] = load8_bf16<TI>(in + (size_t)t * in_ld + (size_t)h * in_hs + k, K - k, a_vec && (k % kIn) == 0);
            const int rb = i / (kHlmTile / 8), cb = (i % (kHlmTile / 8)) * 8;   // an input channel's piece of 8 output channels
            const int kb = k0 + rb, n = n0 + cb;
            bv[j] = make_uint4(0u, 0u, 0u, 0u);
            if (kb < K && n < N) bv[j] = load8_bf16<__nv_bfloat16>(Wh + (size_t)kb * N + n, N - n, b_vec);
        }
        __syncthreads();                                                   // the chunk before is read
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int i = threadIdx.x + j * kHlmThreads;
            *reinterpret_cast<uint4*>(&As[i / (kHlmK / 8)][(i % (kHlmK / 8)) * 8]) = av[j];
            *reinterpret_cast<uint4*>(&Bs[i / (kHlmTile / 8)][(i % (kHlmTile / 8)) * 8]) = bv[j];
        }
        __syncthreads();
        if (!warp_live) continue;
        const int ksteps = min(kHlmK, K - k0 + 15) / 16;                   // the chunk's k-steps that hold channels
        for (int ks = 0; ks < ksteps; ++ks) {
            uint32_t a[4];
            mma_sync::ldmatrix_x4(a, &As[warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                mma_sync::ldmatrix_x4_trans(b, &Bs[ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][np * 16 + (lane >> 4) * 8]);
                mma_sync::mma_bf16(acc[2 * np], a, b[0], b[1]);
                mma_sync::mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
        const int n = n0 + nb * 8 + (lane & 3) * 2;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int t = t0 + warp * 16 + (lane >> 2) + half * 8;
            if (t >= T) continue;
            __nv_bfloat16* dst = out + (size_t)t * out_ld + (size_t)h * out_hs + n;
            float v0 = acc[nb][2 * half], v1 = acc[nb][2 * half + 1];
            if (gate) {
                const float* gr = gate + (size_t)t * gate_ld + (size_t)h * N + n;
                if (n < N) v0 *= 1.0f / (1.0f + expf(-gr[0]));
                if (n + 1 < N) v1 *= 1.0f / (1.0f + expf(-gr[1]));
            }
            if (n < N) dst[0] = __float2bfloat16(v0);
            if (n + 1 < N) dst[1] = __float2bfloat16(v1);
        }
    }
    if (R > 0 && blockIdx.z == 0) {
        for (int i = threadIdx.x; i < nt * (R >> 1); i += kHlmThreads) {
            const int tt = i / (R >> 1), p = i % (R >> 1);
            const TI* src = in + (size_t)(t0 + tt) * in_ld + (size_t)h * in_hs + K;
            float sn, cs;
            sincosf((float)positions[t0 + tt] * freq[p], &sn, &cs);
            sn *= amp;
            cs *= amp;
            const float u = forge::to_float(src[2 * p]), v = forge::to_float(src[2 * p + 1]);
            __nv_bfloat16* dst = out + (size_t)(t0 + tt) * out_ld + (size_t)h * out_hs + N;
            dst[2 * p] = __float2bfloat16(u * cs - v * sn);
            dst[2 * p + 1] = __float2bfloat16(v * cs + u * sn);
        }
    }
}

constexpr int kAttThreads = 256;

// One CTA per (tile of up to TQ consecutive tokens of one request, group of HG heads); tile_t0 = null: tile i is token i.
// A "row" is one (token, head of the group): row = tq * HG + hh.  q [T, H, KD] (KD = C + R), cache rows of KD, out [T, H, C].
template <typename TC>
__global__ void __launch_bounds__(kAttThreads)
latent_attention_kernel(const TC* __restrict__ q, const TC* __restrict__ cache, const int32_t* __restrict__ block_table,
                        const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ tile_t0, const int32_t* __restrict__ tile_n, TC* __restrict__ out, int H, int HG,
                        int C, int R, int page_size, int max_pages, float scale, int TQ, int KT, int window, const float* __restrict__ sink) {
    extern __shared__ float smem[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t0 = tile_t0 ? tile_t0[blockIdx.x] : blockIdx.x;
    const int nq = tile_n ? tile_n[blockIdx.x] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int h0 = blockIdx.y * HG, nh = min(HG, H - h0);
    const int KD = C + R, KP = KD + 1;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    const int max_rows = TQ * HG, rows = nq * nh;
    float* qs = smem;                         // [rows][KD]  queries, already scaled
    float* acc = qs + max_rows * KD;          // [rows][C]   sums of weighted latents
    float* ks = acc + max_rows * C;           // [KT][KD+1]  rows of the chunk
    float* sc = ks + KT * KP;                 // [rows][KT]  scores, then weights
    float* ms = sc + max_rows * KT;           // [rows]      running maximum
    float* ls = ms + max_rows;                // [rows]      running sum
    float* al = ls + max_rows;                // [rows]      what the chunk multiplies the sums so far with
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kAttThreads >> 5;

    for (int i = tid; i < rows * KD; i += kAttThreads) {
        const int d = i % KD, row = i / KD, hh = row % nh, tq = row / nh;
        qs[i] = forge::to_float(q[((size_t)(t0 + tq) * H + h0 + hh) * KD + d]) * scale;
    }
    for (int i = tid; i < rows * C; i += kAttThreads) acc[i] = 0.f;
    for (int i = tid; i < rows; i += kAttThreads) { ms[i] = -INFINITY; ls[i] = 0.f; }

    // chunks of rows that lie behind the window of every token of the tile are skipped: they would add exact zeros
    for (int j0 = (window > 0 ? max(0, pos0 - window + 1) : 0) / KT * KT; j0 <= pos_last; j0 += KT) {
        __syncthreads();                                  // the chunk before is done with ks and sc
        for (int i = tid; i < KT * KD; i += kAttThreads) {
            const int c = i % KD, jj = i / KD, j = j0 + jj;
            float x = 0.f;
            if (j <= pos_last) {
                const int page = table[j / page_size];
                if (page >= 0 && FORGE_PAGE_OK(page)) x = forge::to_float(cache[((size_t)page * page_size + j % page_size) * KD + c]);
            }
            ks[jj * KP + c] = x;
        }
        __syncthreads();
        for (int i = tid; i < rows * KT; i += kAttThreads) {
            const int jj = i % KT, row = i / KT, tq = row / nh;
            float s = -INFINITY;
            if (j0 + jj <= pos0 + tq && (window <= 0 || pos0 + tq - (j0 + jj) < window)) {
                const float* qr = qs + row * KD;
                const float* kr = ks + jj * KP;
                s = 0.f;
                for (int d = 0; d < KD; ++d) s = fmaf(qr[d], kr[d], s);
            }
            sc[i] = s;
        }
        __syncthreads();
        // a warp per row: the chunk's maximum, the weights against the new running maximum, the running sum
        for (int row = warp; row < rows; row += nwarps) {
            float cm = -INFINITY;
            for (int jj = lane; jj < KT; jj += 32) cm = fmaxf(cm, sc[row * KT + jj]);
            cm = forge::warp_max(cm);
            if (cm == -INFINITY) {                        // the token sees nothing of this chunk
                for (int jj = lane; jj < KT; jj += 32) sc[row * KT + jj] = 0.f;
                if (lane == 0) al[row] = 1.f;
                continue;
            }
            const float m_old = ms[row], m_new = fmaxf(m_old, cm);
            float sum = 0.f;
            for (int jj = lane; jj < KT; jj += 32) {
                const float p = expf(sc[row * KT + jj] - m_new);
                sc[row * KT + jj] = p;
                sum += p;
            }
            sum = forge::warp_sum(sum);
            if (lane == 0) {
                al[row] = expf(m_old - m_new);
                ls[row] = ls[row] * al[row] + sum;
                ms[row] = m_new;
            }
        }
        __syncthreads();
        for (int i = tid; i < rows * C; i += kAttThreads) {
            const int c = i % C, row = i / C;
            const float* wr = sc + row * KT;
            const float* vr = ks + c;
            float a = 0.f;
            for (int jj = 0; jj < KT; ++jj) a = fmaf(wr[jj], vr[jj * KP], a);
            acc[i] = fmaf(acc[i], al[row], a);
        }
    }
    __syncthreads();
    for (int i = tid; i < rows * C; i += kAttThreads) {
        const int c = i % C, row = i / C, hh = row % nh, tq = row / nh;
        // a sink joins the denominator as one more weight, exp(sink_h), that has no row of its own
        const float den = sink ? ls[row] + expf(sink[h0 + hh] - ms[row]) : ls[row];
        out[((size_t)(t0 + tq) * H + h0 + hh) * C + c] = forge::from_float<TC>(acc[i] / den);
    }
}

size_t latent_smem_bytes(int HG, int C, int R, int TQ, int KT) {
    const size_t rows = (size_t)TQ * HG;
    return sizeof(float) * (rows * (2 * C + R + KT + 3) + (size_t)KT * (C + R + 1));
}

forge::PerDeviceFlag g_latent_attr[2];

template <typename TI, typename TW, typename TO>
cudaError_t launch_head_linear(cudaStream_t stream, const void* in, long long in_ld, int in_hs, const void* W, void* out, long long out_ld,
                               int out_hs, const int32_t* positions, const float* freq, float amp, int T, int H, int K, int N, int R, const float* gate,
                               long long gate_ld) {
    const dim3 grid((T + kLinTokens - 1) / kLinTokens, H, (N + kLinThreads - 1) / kLinThreads);
    return forge::launch(head_linear_kernel<TI, TW, TO>, grid, dim3(kLinThreads), sizeof(float) * kLinTokens * K, stream, 1, (const TI*)in,
                         in_ld, in_hs, (const TW*)W, (TO*)out, out_ld, out_hs, positions, freq, amp, T, K, N, R, gate, gate_ld);
}

}  // namespace

// proj fp32 [T, ld]: Cq channels of the query's down-projection, then (C > 0) C + R of the key/value one.  wq fp32 [Cq],
// wc fp32 [C]; freq fp32 [R/2].  cq_out [T, Cq] and cache (rows of C + R, row = slot) of type dtype.  slot_mapping null
// or C = 0: nothing stored.
extern "C" int forge_latent_prepare(const float* proj, int ld, const int32_t* positions, const int32_t* slot_mapping, const float* freq,
                                    float amp, const float* wq, const float* wc, void* cq_out, void* cache, int dtype, int T, int Cq,
                                    int C, int R, float eps, cudaStream_t stream) {
    if (T < 0 || Cq <= 0 || C < 0 || R < 0 || (R & 1) || ld < Cq + (C > 0 ? C + R : 0))
        return forge::fail(FORGE_ERR_ARG, "latent_prepare: bad sizes T=%d Cq=%d C=%d R=%d ld=%d", T, Cq, C, R, ld);
    if (C > 0 && slot_mapping && (!cache || !wc || (R > 0 && !freq))) return forge::fail(FORGE_ERR_ARG, "latent_prepare: the cache write needs its tensors");
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(latent_prepare_kernel<TT>, dim3(T), dim3(kPrepThreads), 0, stream, 1, proj, ld, positions, slot_mapping, freq, amp, wq,
                          wc, (TT*)cq_out, (TT*)cache, Cq, C, R, eps));
    return forge::check_launch("latent_prepare", e);
}

// out[t, h, 0:N] = sum_k in[t, h, k] W[h, k, n], and (R > 0) out[t, h, N:N+R] = in[t, h, K:K+R] rotated by positions[t].
// in of in_dtype (fp32 or bf16), W and out of dtype; leading dimensions and head strides in elements.  bf16 weights go to the
// tensor cores (fp32 inputs rounded to bfloat16 on the way) unless `simt` asks for the fp32 multiply-adds.  gate fp32 (rows of
// gate_ld, head h's N numbers from h * N) or null: out[t, h, n] is multiplied by sigmoid(gate[t, h, n]).
extern "C" int forge_head_linear(const void* in, int in_dtype, long long in_ld, int in_hs, const void* W, void* out, int dtype,
                                 long long out_ld, int out_hs, const int32_t* positions, const float* freq, float amp, int T, int H,
                                 int K, int N, int R, int simt, const float* gate, long long gate_ld, cudaStream_t stream) {
    if (T < 0 || H <= 0 || K <= 0 || N <= 0 || R < 0 || (R & 1)) return forge::fail(FORGE_ERR_ARG, "head_linear: bad sizes T=%d H=%d K=%d N=%d R=%d", T, H, K, N, R);
    if (R > 0 && (!positions || !freq)) return forge::fail(FORGE_ERR_ARG, "head_linear: a rotation needs positions and frequencies");
    if (T == 0) return FORGE_OK;
    cudaError_t e;
    if (dtype == FORGE_BF16 && (in_dtype == FORGE_F32 || in_dtype == FORGE_BF16) && !simt) {
        const dim3 grid((T + kHlmTile - 1) / kHlmTile, H, (N + kHlmTile - 1) / kHlmTile);
        if (in_dtype == FORGE_F32)
            e = forge::launch(head_linear_mma_kernel<float>, grid, dim3(kHlmThreads), 0, stream, 1, (const float*)in, in_ld, in_hs,
                              (const __nv_bfloat16*)W, (__nv_bfloat16*)out, out_ld, out_hs, positions, freq, amp, T, K, N, R, gate, gate_ld);
        else
            e = forge::launch(head_linear_mma_kernel<__nv_bfloat16>, grid, dim3(kHlmThreads), 0, stream, 1, (const __nv_bfloat16*)in, in_ld, in_hs,
                              (const __nv_bfloat16*)W, (__nv_bfloat16*)out, out_ld, out_hs, positions, freq, amp, T, K, N, R, gate, gate_ld);
        return forge::check_launch("head_linear (tensor cores)", e);
    }
    if (sizeof(float) * kLinTokens * K > 48 * 1024) return forge::fail(FORGE_ERR_UNSUPPORTED, "head_linear: %d input channels a head", K);
    if (dtype == FORGE_F32 && in_dtype == FORGE_F32)
        e = launch_head_linear<float, float, float>(stream, in, in_ld, in_hs, W, out, out_ld, out_hs, positions, freq, amp, T, H, K, N, R, gate, gate_ld);
    else if (dtype == FORGE_BF16 && in_dtype == FORGE_F32)
        e = launch_head_linear<float, __nv_bfloat16, __nv_bfloat16>(stream, in, in_ld, in_hs, W, out, out_ld, out_hs, positions, freq, amp, T, H, K, N, R, gate, gate_ld);
    else if (dtype == FORGE_BF16 && in_dtype == FORGE_BF16)
        e = launch_head_linear<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(stream, in, in_ld, in_hs, W, out, out_ld, out_hs, positions, freq, amp, T, H, K, N, R, gate, gate_ld);
    else
        return forge::fail(FORGE_ERR_ARG, "head_linear: input type %d with weights of type %d", in_dtype, dtype);
    return forge::check_launch("head_linear", e);
}

// Bytes of shared memory of a tile of TQ tokens and HG heads with key chunks of KT (the caller picks TQ and HG with it).
extern "C" long long forge_latent_attention_smem(int HG, int C, int R, int TQ, int KT) { return (long long)latent_smem_bytes(HG, C, R, TQ, KT); }

// q [T, H, C+R], out [T, H, C] and cache (rows of C + R) of type dtype.  tile_t0 / tile_n int32 [num_tiles] (both null: one
// token a tile).  HG: heads per CTA.  window: position i reads the rows j with i - window < j <= i (0: every j <= i);
// sink fp32 [H] or null: exp(sink_h) is added to head h's softmax denominator.
extern "C" int forge_latent_attention(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                      const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, void* out, int dtype,
                                      int num_tiles, int H, int HG, int C, int R, int page_size, int max_pages, float scale, int TQ,
                                      int KT, int window, const float* sink, cudaStream_t stream) {
    if (num_tiles < 0 || H <= 0 || HG <= 0 || C <= 0 || R < 0 || page_size <= 0 || max_pages <= 0 || TQ <= 0 || KT <= 0)
        return forge::fail(FORGE_ERR_ARG, "latent_attention: bad sizes tiles=%d H=%d HG=%d C=%d R=%d page=%d TQ=%d KT=%d", num_tiles, H, HG, C,
                           R, page_size, TQ, KT);
    if ((tile_t0 == nullptr) != (tile_n == nullptr)) return forge::fail(FORGE_ERR_ARG, "latent_attention: half a tile list");
    if (num_tiles == 0) return FORGE_OK;
    const size_t smem = latent_smem_bytes(HG, C, R, TQ, KT);
    if (smem > 200 * 1024)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "latent_attention: a tile of %d tokens, %d heads and %d keys needs %zu bytes of shared memory", TQ, HG, KT, smem);
    bool& done = g_latent_attr[dtype == FORGE_BF16].current();
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT, {
        if (!done) {
            e = cudaFuncSetAttribute(latent_attention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return forge::check_launch("latent_attention (shared memory)", e);
            done = true;
        }
        e = forge::launch(latent_attention_kernel<TT>, dim3(num_tiles, (H + HG - 1) / HG), dim3(kAttThreads), smem, stream, 1, (const TT*)q,
                          (const TT*)cache, block_table, tok_req, positions, tile_t0, tile_n, (TT*)out, H, HG, C, R, page_size, max_pages, scale,
                          TQ, KT, window, sink);
    });
    return forge::check_launch("latent_attention", e);
}

FORGE_DEFINE_CHECKS_ENTRY(attention_latent)

extern "C" const char* forge_last_error() { return forge::error_buffer(); }
