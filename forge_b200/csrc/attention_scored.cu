// Causal softmax attention over the paged cache whose SCORES are shaped by options, and the step that prepares its
// operands.  Each option is a parameter, so one kernel serves several mixers:
//
//   maps M      a head's query and a key/value head's key are M vectors of D channels ("maps"); each map is a softmax
//               of its own over the same values.  M = 1: ordinary attention.  M = 2 (differential attention):
//                   o = a_1 - lambda a_2,   o <- o / sqrt(mean(o^2) + eps) * post          (a_m: map m's output)
//   distance    score(i, j) = scale q(i) . k(j) - r1_h ln(1 + r2_h (i - j))     (r1 = null: no such term)
//   out_scale   the head outputs are multiplied by it (a mixer that runs beside another one with weights of their own)
//   window      position i sees j only if i - j < window                              (0: no such limit)
//   chunk       position i sees j only if i / chunk == j / chunk (integer division)     (0: no such limit)
//   softcap     score <- softcap tanh(score / softcap), after the scale                (0: none)
//
// and in the prepare step:  an RMS norm over ALL of a token's query channels (and all of its key channels) with a
// weight per channel; a query temperature 1 + coef ln(floor((p + 1) / every) + 1) at position p; a rotation of the first
// rot_dims channels of every map, channel i paired with i + rot_dims/2.
//
// Query heads have M*D channels, key heads M*D, value heads E; a cache page is [kv head][token in page][M*D] keys followed
// by [kv head][token in page][E] values.  All arithmetic is fp32 whatever the storage type.  Keys are walked in chunks of KT
// positions that start at multiples of KT, a chunk's weights are summed in a fixed order, and a key that a token does not
// see adds exact zeros: what a token adds up, and in which order, depends on its position alone, not on the step's cut, the
// tile, or the batch around it.
#include "common.cuh"
#include "checks.cuh"

namespace {

constexpr int kPrepThreads = 256;

// One CTA per token, or (steps of few tokens) several that share a token's channels; each of them takes the norms' sums over
// the whole row, which is cheaper than a second launch.  proj fp32 row = [q: QU units of D | k: KU units of D | v: G heads of E].
template <typename TC>
__global__ void __launch_bounds__(kPrepThreads)
scored_prepare_kernel(const float* __restrict__ proj, int ld, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                      const float* __restrict__ q_norm, const float* __restrict__ k_norm, TC* __restrict__ q_out,
                      TC* __restrict__ cache, int QU, int KU, int G, int D, int E, int rot_dims, float eps, float temp_coef,
                      float temp_every, int page_size, long long page_stride) {
    __shared__ float red[32];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const int ipos = positions[t];
    const float pos = (float)ipos;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const bool store = slot >= 0 && FORGE_SLOT_OK(slot);
    const int page = store ? slot / page_size : 0, off = store ? slot % page_size : 0;
    const int QW = QU * D, KW = KU * D, KD = KW / G;
    TC* kbase = cache + (size_t)page * page_stride;
    TC* vbase = kbase + (size_t)G * page_size * KD;
    float inv_q = 1.f, inv_k = 1.f;
    if (q_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < QW; c += kPrepThreads) ss = fmaf(row[c], row[c], ss);
        inv_q = 1.0f / sqrtf(forge::block_sum(ss, red) / (float)QW + eps);
    }
    if (k_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < KW; c += kPrepThreads) ss = fmaf(row[QW + c], row[QW + c], ss);
        inv_k = 1.0f / sqrtf(forge::block_sum(ss, red) / (float)KW + eps);
    }
    const float temp = temp_every > 0.f ? 1.0f + temp_coef * logf(floorf((pos + 1.0f) / temp_every) + 1.0f) : 1.0f;
    const int half = rot_dims >> 1;
    auto value = [&](int idx) {          // the channel after its norm
        float x = row[idx];
        if (idx < QW) { if (q_norm) x = x * inv_q * q_norm[idx]; }
        else if (k_norm) x = x * inv_k * k_norm[idx - QW];
        return x;
    };
    const int first = blockIdx.y * kPrepThreads + threadIdx.x, step = gridDim.y * kPrepThreads;
    for (int idx = first; idx < QW + KW; idx += step) {
        const int d = idx % D;
        float x = value(idx);
        if (d < rot_dims) {
            float s, c;
            sincosf(pos * inv_freq[d < half ? d : d - half], &s, &c);
            x = d < half ? x * c - value(idx + half) * s : x * c + value(idx - half) * s;
        }
        if (idx < QW) {
            q_out[(size_t)t * QW + idx] = forge::from_float<TC>(x * temp);
        } else if (store) {
            const int c = idx - QW;
            kbase[((size_t)(c / KD) * page_size + off) * KD + c % KD] = forge::from_float<TC>(x);
        }
    }
    if (store)
        for (int idx = first; idx < G * E; idx += step)
            vbase[((size_t)(idx / E) * page_size + off) * E + idx % E] = forge::from_float<TC>(row[QW + KW + idx]);
}

constexpr int kAttThreads = 256;

// The first position that position `pos` sees.  It does not fall as pos grows.
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
    int lo = 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

// One CTA per (tile of up to TQ consecutive tokens of one request, key/value head); tile_t0 = null: tile i is token i.
// A "row" is one (token, query head of this kv head, map): row = (tq * R + r) * M + m.
template <typename TC>
__global__ void __launch_bounds__(kAttThreads)
scored_attention_kernel(const TC* __restrict__ q, const TC* __restrict__ cache, const int32_t* __restrict__ block_table,
                        const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ tile_t0, const int32_t* __restrict__ tile_n, const float* __restrict__ r1,
                        const float* __restrict__ r2, TC* __restrict__ out, int H, int G, int M, int D, int E, int page_size,
                        long long page_stride, int max_pages, float scale, float lambda, float post, float eps, float out_scale,
                        int TQ, int KT, long long out_ld, int window, int chunk, float softcap) {
    extern __shared__ float smem[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int t0 = tile_t0 ? tile_t0[blockIdx.x] : blockIdx.x;
    const int nq = tile_n ? tile_n[blockIdx.x] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int g = blockIdx.y, R = H / G, KD = M * D, KP = KD + 1;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    const int max_rows = TQ * R * M, rows = nq * R * M;
    float* qs = smem;                         // [rows][D]   queries, already scaled
    float* acc = qs + max_rows * D;           // [rows][E]   outputs being added up
    float* ks = acc + max_rows * E;           // [KT][KD+1]  keys of the chunk
    float* vs = ks + KT * KP;                 // [KT][E]     values of the chunk
    float* sc = vs + KT * E;                  // [rows][KT]  scores, then weights
    float* ms = sc + max_rows * KT;           // [rows]      running maximum
    float* ls = ms + max_rows;                // [rows]      running sum
    float* al = ls + max_rows;                // [rows]      what the chunk multiplies the sums so far with
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kAttThreads >> 5;
    const size_t q_ld = (size_t)H * KD;

    for (int i = tid; i < rows * D; i += kAttThreads) {
        const int d = i % D, row = i / D, m = row % M, r = (row / M) % R, tq = row / (M * R);
        qs[i] = forge::to_float(q[(size_t)(t0 + tq) * q_ld + ((size_t)(g * R + r) * M + m) * D + d]) * scale;
    }
    for (int i = tid; i < rows * E; i += kAttThreads) acc[i] = 0.f;
    for (int i = tid; i < rows; i += kAttThreads) { ms[i] = -INFINITY; ls[i] = 0.f; }

    const TC* vcache = cache + (size_t)G * page_size * KD;
    // chunks of keys that no token of the tile sees are skipped: they would add exact zeros
    for (int j0 = first_visible(pos0, window, chunk) / KT * KT; j0 <= pos_last; j0 += KT) {
        __syncthreads();                                  // the chunk before is done with ks, vs, sc
        for (int i = tid; i < KT * KD; i += kAttThreads) {
            const int c = i % KD, jj = i / KD, j = j0 + jj;
            float x = 0.f;
            if (j <= pos_last) {
                const int page = table[j / page_size];
                if (page >= 0 && FORGE_PAGE_OK(page))
                    x = forge::to_float(cache[(size_t)page * page_stride + ((size_t)g * page_size + j % page_size) * KD + c]);
            }
            ks[jj * KP + c] = x;
        }
        for (int i = tid; i < KT * E; i += kAttThreads) {
            const int e = i % E, jj = i / E, j = j0 + jj;
            float x = 0.f;
            if (j <= pos_last) {
                const int page = table[j / page_size];
                if (page >= 0 && FORGE_PAGE_OK(page))
                    x = forge::to_float(vcache[(size_t)page * page_stride + ((size_t)g * page_size + j % page_size) * E + e]);
            }
            vs[i] = x;
        }
        __syncthreads();
        for (int i = tid; i < rows * KT; i += kAttThreads) {
            const int jj = i % KT, row = i / KT, m = row % M, r = (row / M) % R, tq = row / (M * R);
            const int pos = pos0 + tq, j = j0 + jj;
            float s = -INFINITY;
            if (j <= pos && j >= first_visible(pos, window, chunk)) {
                const float* qr = qs + row * D;
                const float* kr = ks + jj * KP + m * D;
                s = 0.f;
                for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
                if (r1) s -= r1[g * R + r] * log1pf(r2[g * R + r] * (float)(pos - j));
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
                const float a = expf(m_old - m_new);
                al[row] = a;
                ls[row] = ls[row] * a + sum;
                ms[row] = m_new;
            }
        }
        __syncthreads();
        for (int i = tid; i < rows * E; i += kAttThreads) {
            const int e = i % E, row = i / E;
            const float* wr = sc + row * KT;
            const float* vr = vs + e;
            float a = 0.f;
            for (int jj = 0; jj < KT; ++jj) a = fmaf(wr[jj], vr[jj * E], a);
            acc[i] = fmaf(acc[i], al[row], a);
        }
    }
    __syncthreads();
    if (M == 1) {
        for (int i = tid; i < rows * E; i += kAttThreads) {
            const int e = i % E, row = i / E, r = row % R, tq = row / R;
            out[(size_t)(t0 + tq) * out_ld + (size_t)(g * R + r) * E + e] = forge::from_float<TC>(acc[i] / ls[row] * out_scale);
        }
        return;
    }
    // two maps: a warp per (token, head) takes o = a_1 - lambda a_2, divides it by its root mean square, scales it
    for (int pr = warp; pr < nq * R; pr += nwarps) {
        const int r = pr % R, tq = pr / R;
        const float* a1 = acc + (size_t)(pr * 2) * E;
        const float* a2 = a1 + E;
        const float l1 = ls[pr * 2], l2 = ls[pr * 2 + 1];
        float ss = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float o = a1[e] / l1 - lambda * (a2[e] / l2);
            ss = fmaf(o, o, ss);
        }
        ss = forge::warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)E + eps) * post * out_scale;
        for (int e = lane; e < E; e += 32)
            out[(size_t)(t0 + tq) * out_ld + (size_t)(g * R + r) * E + e] = forge::from_float<TC>((a1[e] / l1 - lambda * (a2[e] / l2)) * inv);
    }
}

size_t scored_smem_bytes(int R, int M, int D, int E, int TQ, int KT) {
    const size_t rows = (size_t)TQ * R * M;
    return sizeof(float) * (rows * (D + E + KT + 3) + (size_t)KT * (M * D + 1 + E));
}

forge::PerDeviceFlag g_scored_attr[2];

}  // namespace

// proj fp32 [T, ld]: per row QU query units of D channels, KU key units of D (KU / G consecutive ones are a key/value
// head's key), G value heads of E.  inv_freq fp32 [rot_dims / 2] (null with rot_dims 0).  q_norm fp32 [QU*D], k_norm fp32
// [KU*D] or null.  temp_every <= 0: no temperature.  cache: pages of page_stride elements; slot_mapping null: nothing stored.
extern "C" int forge_scored_prepare(const float* proj, int ld, const int32_t* positions, const int32_t* slot_mapping,
                                    const float* inv_freq, const float* q_norm, const float* k_norm, void* q_out, void* cache,
                                    int dtype, int T, int QU, int KU, int G, int D, int E, int rot_dims, float eps, float temp_coef,
                                    float temp_every, int page_size, long long page_stride, cudaStream_t stream) {
    if (T < 0 || QU <= 0 || KU <= 0 || G <= 0 || D <= 0 || E <= 0 || KU % G != 0 || page_size <= 0 || rot_dims < 0 || rot_dims > D ||
        (rot_dims & 1))
        return forge::fail(FORGE_ERR_ARG, "scored_prepare: bad sizes T=%d QU=%d KU=%d G=%d D=%d E=%d rot=%d page=%d", T, QU, KU, G, D, E,
                           rot_dims, page_size);
    if (rot_dims > 0 && !inv_freq) return forge::fail(FORGE_ERR_ARG, "scored_prepare: a rotation needs its frequencies");
    if (ld < (QU + KU) * D + G * E) return forge::fail(FORGE_ERR_ARG, "scored_prepare: rows of %d are too short", ld);
    if (slot_mapping && (!cache || page_stride < (long long)page_size * (KU * D + G * E)))
        return forge::fail(FORGE_ERR_ARG, "scored_prepare: pages are too small");
    if (T == 0) return FORGE_OK;
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT,
        e = forge::launch(scored_prepare_kernel<TT>, dim3(T, T >= 256 ? 1 : min(16, ((QU + KU) * D + 511) / 512)), dim3(kPrepThreads), 0, stream, 1, proj, ld, positions, slot_mapping,
                          inv_freq, q_norm, k_norm, (TT*)q_out, (TT*)cache, QU, KU, G, D, E, rot_dims, eps, temp_coef, temp_every,
                          page_size, page_stride));
    return forge::check_launch("scored_prepare", e);
}

// Bytes of shared memory of a tile of TQ tokens with key chunks of KT (the caller picks TQ with it).
extern "C" long long forge_scored_attention_smem(int H, int G, int M, int D, int E, int TQ, int KT) {
    return (long long)scored_smem_bytes(H / (G > 0 ? G : 1), M, D, E, TQ, KT);
}

// q [T, H*M*D] and out (rows of out_ld elements, the heads' H*E values at their start) in the cache's type.  tile_t0 / tile_n int32 [num_tiles] (both null: one token a tile).
// r1, r2 fp32 [H] or both null.  M = 2: lambda, post and eps of the combination of the two maps.  window, chunk, softcap: 0 = none.
extern "C" int forge_scored_attention(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                      const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, const float* r1,
                                      const float* r2, void* out, int dtype, int num_tiles, int H, int G, int M, int D, int E,
                                      int page_size, long long page_stride, int max_pages, float scale, float lambda, float post,
                                      float eps, float out_scale, int TQ, int KT, long long out_ld, int window, int chunk, float softcap,
                                      cudaStream_t stream) {
    if (out_ld < (long long)H * E) return forge::fail(FORGE_ERR_ARG, "scored_attention: output rows of %lld are too short", out_ld);
    if (num_tiles < 0 || H <= 0 || G <= 0 || D <= 0 || E <= 0 || H % G != 0 || (M != 1 && M != 2) || page_size <= 0 || max_pages <= 0 ||
        TQ <= 0 || KT <= 0)
        return forge::fail(FORGE_ERR_ARG, "scored_attention: bad sizes tiles=%d H=%d G=%d M=%d D=%d E=%d page=%d TQ=%d KT=%d", num_tiles,
                           H, G, M, D, E, page_size, TQ, KT);
    if ((tile_t0 == nullptr) != (tile_n == nullptr)) return forge::fail(FORGE_ERR_ARG, "scored_attention: half a tile list");
    if ((r1 == nullptr) != (r2 == nullptr)) return forge::fail(FORGE_ERR_ARG, "scored_attention: r1 and r2 go together");
    if (window < 0 || chunk < 0 || softcap < 0.f) return forge::fail(FORGE_ERR_ARG, "scored_attention: window %d, chunk %d, softcap %g", window, chunk, (double)softcap);
    if (num_tiles == 0) return FORGE_OK;
    const size_t smem = scored_smem_bytes(H / G, M, D, E, TQ, KT);
    if (smem > 200 * 1024)
        return forge::fail(FORGE_ERR_UNSUPPORTED, "scored_attention: a tile of %d tokens and %d keys needs %zu bytes of shared memory", TQ, KT, smem);
    bool& done = g_scored_attr[dtype == FORGE_BF16].current();
    cudaError_t e = cudaSuccess;
    FORGE_DISPATCH_DTYPE(dtype, TT, {
        if (!done) {
            e = cudaFuncSetAttribute(scored_attention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return forge::check_launch("scored_attention (shared memory)", e);
            done = true;
        }
        e = forge::launch(scored_attention_kernel<TT>, dim3(num_tiles, G), dim3(kAttThreads), smem, stream, 1, (const TT*)q,
                          (const TT*)cache, block_table, tok_req, positions, tile_t0, tile_n, r1, r2, (TT*)out, H, G, M, D, E, page_size,
                          page_stride, max_pages, scale, lambda, post, eps, out_scale, TQ, KT, out_ld, window, chunk, softcap);
    });
    return forge::check_launch("scored_attention", e);
}

FORGE_DEFINE_CHECKS_ENTRY(attention_scored)
